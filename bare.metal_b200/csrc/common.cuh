// Shared device helpers: 128-bit vector access for fp32 / bf16 activations and warp reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace bmb {

typedef __nv_bfloat16 bf16;

// Function attributes (cudaFuncSetAttribute) and the SM count belong to a device, not to the process: a launcher keeps one
// mask per set-up site and repeats the set-up the first time it runs with another device current. Setting an attribute
// twice is harmless, so two host threads racing through the same first use need no lock.
inline bool first_use_on_current_device(std::atomic<unsigned long long>& done_mask) {
    int dev = 0;
    cudaGetDevice(&dev);
    const unsigned long long bit = 1ull << (dev & 63);
    if (done_mask.load(std::memory_order_acquire) & bit) return false;
    done_mask.fetch_or(bit, std::memory_order_acq_rel);
    return true;
}
inline int sm_count_current_device() {
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    int n = cached[dev & 63].load(std::memory_order_relaxed);
    if (n == 0) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev & 63].store(n, std::memory_order_relaxed);
    }
    return n;
}

// One 16-byte vector of T, processed as floats.
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ __forceinline__ static void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    __device__ __forceinline__ static void store(float* p, const float (&f)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
    // the 16 bytes as loaded, for kernels that keep several vectors in flight and widen them only when used
    using Raw = uint4;
    __device__ __forceinline__ static Raw load_raw(const float* p) { return *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ static void unpack(const Raw& v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
};
template <> struct Vec<bf16> {
    static constexpr int N = 8;
    __device__ __forceinline__ static void load(const bf16* p, float (&f)[8]) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
    __device__ __forceinline__ static void store(bf16* p, const float (&f)[8]) {
        uint4 v;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = v;
    }
    using Raw = uint4;
    __device__ __forceinline__ static Raw load_raw(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ static void unpack(const Raw& v, float (&f)[8]) {
        f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
        f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
        f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
        f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
    }
};

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace bmb

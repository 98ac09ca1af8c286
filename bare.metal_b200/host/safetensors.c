/* HF safetensors directory loader — placeholder until the weights-directory reader is built. */
#include <stdio.h>
#include "bm_internal.h"
int bm_load_safetensors_dir(bm_model_t* m, const char* dir) { (void)m; (void)dir; return -1; }

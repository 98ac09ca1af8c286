#include <stdio.h>
int main(void) { fprintf(stderr, "baremetal-train: not built yet\n"); return 2; }

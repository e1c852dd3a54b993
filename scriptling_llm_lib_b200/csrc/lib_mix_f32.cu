// Kernels of latent attention, decayed linear attention, the selective scan, routed experts and the norm without
// statistics, true 32-bit set.
#include "mix_kernels.cuh"
#define ELEM float
#define FN(name) sllm_##name##_f32
#include "mix_launchers.inc"

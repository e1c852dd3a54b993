// Kernels of latent attention, decayed linear attention, the selective scan, routed experts and the norm without
// statistics on bfloat16 activations and weights (float state and sums).
#include "mix_kernels.cuh"
#define ELEM bf16
#define FN(name) sllm_##name##_bf16
#include "mix_launchers.inc"

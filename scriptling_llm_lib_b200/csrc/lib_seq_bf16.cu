// Kernels of the mixers with state along the sequence on bfloat16 activations and weights (float state and sums).
#include "sequence_kernels.cuh"
#define ELEM bf16
#define FN(name) sllm_##name##_bf16
#include "sequence_launchers.inc"

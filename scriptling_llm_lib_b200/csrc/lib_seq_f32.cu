// Kernels of the mixers with state along the sequence, true 32-bit set.
#include "sequence_kernels.cuh"
#define ELEM float
#define FN(name) sllm_##name##_f32
#include "sequence_launchers.inc"

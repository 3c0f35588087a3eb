// The true 32-bit kernel set: float weights, float activations, FP32 FMA accumulation.
#include "generic_kernels.cuh"
#define ELEM float
#define FN(name) sllm_##name##_f32
#include "generic_launchers.inc"

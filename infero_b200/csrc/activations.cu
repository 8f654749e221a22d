// Activations of feed-forward layers that are not fused into a product's epilogue.
//
//   glu:   out[t, j] = glu_act(v[t, 2j], v[t, 2j + 1])   gate and up alternate along a row (the layout of the stacked
//          gate/up products); the gated activations are those of common.cuh
//   relu2: out[t, j] = max(v[t, j], 0)^2
// v is a tensor of the step's element type or `splits` 32-bit partial sums of a product (added in ascending order);
// the arithmetic is 32-bit.
#include "common.cuh"

namespace {

template <typename TI>
__device__ __forceinline__ float summed(const TI* __restrict__ v, int splits, long long split_stride, size_t at) {
    float s = to_f32(v[at]);
    for (int k = 1; k < splits; ++k) s += to_f32(v[at + (size_t)k * split_stride]);
    return s;
}

template <typename TI, typename TO>
__global__ void glu_act_kernel(const TI* __restrict__ v, int splits, long long split_stride, TO* __restrict__ out, int ff,
                               size_t total, int kind, float limit, float alpha) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / ff, j = i % ff;
    const size_t at = t * 2 * ff + 2 * j;
    out[i] = from_f32<TO>(glu_act(summed(v, splits, split_stride, at), summed(v, splits, split_stride, at + 1), kind, limit, alpha));
}

template <typename TI, typename TO>
__global__ void relu2_kernel(const TI* __restrict__ v, int splits, long long split_stride, TO* __restrict__ out, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float x = fmaxf(summed(v, splits, split_stride, i), 0.f);
    out[i] = from_f32<TO>(x * x);
}

}  // namespace

extern "C" {

#define DISPATCH(KERNEL, ...)                                                                                      \
    do {                                                                                                           \
        if (in_dtype == INFERO_F32 && out_dtype == INFERO_F32) KERNEL<float, float><<<blocks, 256, 0, stream>>>((const float*)v, splits, split_stride, (float*)out, __VA_ARGS__); \
        else if (in_dtype == INFERO_F32) KERNEL<float, bf16><<<blocks, 256, 0, stream>>>((const float*)v, splits, split_stride, (bf16*)out, __VA_ARGS__); \
        else if (out_dtype == INFERO_F32) KERNEL<bf16, float><<<blocks, 256, 0, stream>>>((const bf16*)v, splits, split_stride, (float*)out, __VA_ARGS__); \
        else KERNEL<bf16, bf16><<<blocks, 256, 0, stream>>>((const bf16*)v, splits, split_stride, (bf16*)out, __VA_ARGS__); \
    } while (0)

// v: splits arrays of [n_tokens, 2 * ff], split_stride elements apart; out [n_tokens, ff].
int infero_glu_act(const void* v, int in_dtype, int splits, long long split_stride, void* out, int out_dtype, int n_tokens,
                   int ff, int kind, float limit, float alpha, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * ff;
    if (total == 0) return 0;
    INFERO_REQUIRE(splits >= 1 && (kind == GLU_SILU || kind == GLU_CLAMPED), "glu: %d splits, activation %d", splits, kind);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    DISPATCH(glu_act_kernel, ff, total, kind, limit, alpha);
    return infero_check_launch("glu_act");
}

// v: splits arrays of [n_tokens, ff]; out [n_tokens, ff].
int infero_relu2(const void* v, int in_dtype, int splits, long long split_stride, void* out, int out_dtype, int n_tokens,
                 int ff, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * ff;
    if (total == 0) return 0;
    INFERO_REQUIRE(splits >= 1, "relu2: %d splits", splits);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    DISPATCH(relu2_kernel, total);
    return infero_check_launch("relu2");
}
#undef DISPATCH

}  // extern "C"

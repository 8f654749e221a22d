// Residual update of a layer that normalises a sublayer's *result*, with an elementwise gate in front:
//
//   z = y * sigmoid(g + b)            (the gate's logits g come from a product of the sublayer's input)
//   x += z / sqrt(mean(z^2) + eps) * w     (w one number for all coordinates)
//
// all in 32-bit, one block per token; the new x is also left in the activation type for the products
// of the next sublayer.  Without a gate (g == nullptr) z = y.  A second entry point only converts rows
// of the 32-bit residual stream to the activation type (the input of the first sublayer).
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

// PER > 0: the row's d <= PER * THREADS gated values stay in registers between the two passes
template <int PER>
__global__ void __launch_bounds__(THREADS)
gated_scalar_norm_add_kernel(float* __restrict__ x, const float* __restrict__ y, int y_stride,
                             const float* __restrict__ gate, int gate_stride, const float* __restrict__ gate_bias,
                             const float* __restrict__ norm_w, float eps, bf16* __restrict__ h_out, int d) {
    __shared__ float red[32];
    const size_t t = blockIdx.x;
    const float* yr = y + t * y_stride;
    const float* gr = gate ? gate + t * gate_stride : nullptr;
    auto gated = [&](int i) {
        float z = yr[i];
        if (gr) z *= 1.0f / (1.0f + expf(-(gr[i] + (gate_bias ? gate_bias[i] : 0.f))));
        return z;
    };
    float keep[PER > 0 ? PER : 1];
    float ss = 0.f;
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = k * THREADS + threadIdx.x;
            keep[k] = i < d ? gated(i) : 0.f;
            ss = fmaf(keep[k], keep[k], ss);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += THREADS) {
            const float z = gated(i);
            ss = fmaf(z, z, ss);
        }
    }
    ss = block_sum(ss, red);
    const float r = norm_w[0] / sqrtf(ss / (float)d + eps);
    float* xr = x + t * d;
    if (PER > 0) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = k * THREADS + threadIdx.x;
            if (i < d) {
                const float v = xr[i] + keep[k] * r;
                xr[i] = v;
                if (h_out) h_out[t * d + i] = __float2bfloat16_rn(v);
            }
        }
    } else {
        for (int i = threadIdx.x; i < d; i += THREADS) {
            const float v = xr[i] + gated(i) * r;
            xr[i] = v;
            if (h_out) h_out[t * d + i] = __float2bfloat16_rn(v);
        }
    }
}

__global__ void cast_rows_kernel(const float* __restrict__ x, bf16* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(x[i]);
}

}  // namespace

extern "C" {

int infero_gated_scalar_norm_add(float* x, const float* y, int y_stride, const float* gate, int gate_stride,
                                 const float* gate_bias, const float* norm_w, float eps, void* h_out_bf16,
                                 int n_rows, int d, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    INFERO_REQUIRE(d > 0 && y_stride >= d, "gated norm: bad sizes d=%d stride=%d", d, y_stride);
#define GO(PER_) gated_scalar_norm_add_kernel<PER_><<<n_rows, THREADS, 0, stream>>>(x, y, y_stride, gate, gate_stride, gate_bias, \
                                                                                   norm_w, eps, (bf16*)h_out_bf16, d)
    if (d <= 4 * THREADS) GO(4);
    else if (d <= 8 * THREADS) GO(8);
    else if (d <= 16 * THREADS) GO(16);
    else GO(0);
#undef GO
    return infero_check_launch("gated_scalar_norm_add");
}

int infero_cast_rows_bf16(const float* x, void* out, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    cast_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, (bf16*)out, (size_t)n);
    return infero_check_launch("cast_rows_bf16");
}

}  // extern "C"

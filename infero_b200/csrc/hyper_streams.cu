// Layer norm, and a residual kept as several streams ("hyper-connections").
//
// layer norm (weight, no bias):  h = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w, v = x (+ delta), all
//   32-bit, the variance from the deviations (two passes over the row, which sits in shared memory).
//
// streams: the residual of a token is S vectors xs[s] of width d (float32 [T, S, d]).  A sublayer reads
//   u = sum_s a[s] xs[s], works on h = norm(u), and its result y updates all streams at once from the old ones,
//   xs'[r] = sum_s m[s, r] xs[s] + b[r] y.  One kernel does the update of the sublayer before (if y is given) and the
//   read-out and norm for the sublayer after (if a is given): one pass over a token's streams per sublayer, as
//   the single-stream blocks have one pass for add + norm.  Without a norm weight the read-out is written as it is
//   (float32): the sum of the streams at the end of the model is a read-out with a = 1.
// The small vectors a, b, m are float32 on both precisions.  One block per token; nothing depends on the batch.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;          // per token in steps of many tokens
constexpr int THREADS_FEW = 1024;     // in steps of few tokens, where a block's own latency is what counts
constexpr int MAX_STREAMS = 8;

// the row v[0..d) in shared memory -> out = layer norm(v) * w
template <typename OutT>
__device__ __forceinline__ void layernorm_row(const float* v, const float* __restrict__ w, float eps, OutT* __restrict__ out,
                                              int d, float* red) {
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) s += v[i];
    const float mean = block_sum(s, red) / (float)d;
    float q = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float c = v[i] - mean;
        q = fmaf(c, c, q);
    }
    const float rstd = 1.0f / sqrtf(block_sum(q, red) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = from_f32<OutT>((v[i] - mean) * rstd * w[i]);
}

template <typename OutT>
__global__ void __launch_bounds__(THREADS_FEW)
add_layernorm_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ w, float eps,
                     OutT* __restrict__ out, const int* __restrict__ rows, int d) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const size_t t = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (delta) {
            v += delta[t * d + i];
            if (!rows) xr[i] = v;
        }
        row[i] = v;
    }
    __syncthreads();
    layernorm_row(row, w, eps, out + (size_t)blockIdx.x * d, d, red);
}

template <typename OutT>
__global__ void __launch_bounds__(THREADS_FEW)
hyper_step_kernel(float* __restrict__ xs, const float* __restrict__ y, int y_stride, int y_splits, long long y_split_stride,
                  const float* __restrict__ mix,
                  const float* __restrict__ w_out, const float* __restrict__ w_in, const float* __restrict__ norm_w,
                  float eps, OutT* __restrict__ h_out, float* __restrict__ u_out, const int* __restrict__ rows, int S, int d) {
    extern __shared__ float row[];
    __shared__ float red[32];
    __shared__ float m_s[MAX_STREAMS * MAX_STREAMS], b_s[MAX_STREAMS], a_s[MAX_STREAMS];
    if (threadIdx.x < S * S && y) m_s[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (y) b_s[threadIdx.x] = w_out[threadIdx.x];
        a_s[threadIdx.x] = w_in ? w_in[threadIdx.x] : 1.0f;
    }
    __syncthreads();
    const size_t t = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xt = xs + t * S * d;
    const bool read_out = w_in || u_out || norm_w;       // (without w_in: the plain sum of the streams)
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) v[s] = s < S ? xt[(size_t)s * d + i] : 0.f;
        if (y) {
            float yv = y[t * y_stride + i];
            for (int k = 1; k < y_splits; ++k) yv += y[(size_t)k * y_split_stride + t * y_stride + i];     // ascending order
            float nv[MAX_STREAMS];
#pragma unroll
            for (int r = 0; r < MAX_STREAMS; ++r) {
                float acc = 0.f;
                if (r < S) {
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s)
                        if (s < S) acc = fmaf(m_s[s * S + r], v[s], acc);
                    acc = fmaf(b_s[r], yv, acc);
                    xt[(size_t)r * d + i] = acc;
                }
                nv[r] = acc;
            }
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s) v[s] = nv[s];
        }
        if (read_out) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) u = fmaf(a_s[s], v[s], u);
            if (norm_w) row[i] = u;
            else u_out[(size_t)blockIdx.x * d + i] = u;
        }
    }
    if (!read_out || !norm_w) return;
    __syncthreads();
    layernorm_row(row, norm_w, eps, h_out + (size_t)blockIdx.x * d, d, red);
}

__global__ void streams_fill_kernel(const float* __restrict__ x, float* __restrict__ xs, int S, int d) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = x[t * d + i];
        for (int s = 0; s < S; ++s) xs[(t * S + s) * d + i] = v;
    }
}

}  // namespace

extern "C" {

// x float32 [T, d] (+= delta float32 [T, d] if given; with `rows` x is left as it is); out [n, d] = layer norm of rows.
int infero_add_layernorm(float* x, const float* delta, const float* w, float eps, void* out, int out_dtype,
                         const int* rows, int n, int d, cudaStream_t stream) {
    if (n == 0) return 0;
    const size_t sh = (size_t)d * sizeof(float);
    INFERO_REQUIRE(d >= 1 && sh <= 48 * 1024, "layer norm: width %d outside 1..12288", d);
    const int threads = n <= 64 && d > THREADS ? THREADS_FEW : THREADS;
    if (out_dtype == INFERO_F32)
        add_layernorm_kernel<float><<<n, threads, sh, stream>>>(x, delta, w, eps, (float*)out, rows, d);
    else
        add_layernorm_kernel<bf16><<<n, threads, sh, stream>>>(x, delta, w, eps, (bf16*)out, rows, d);
    return infero_check_launch("add_layernorm");
}

// xs float32 [T, S, d].  y (float32, row stride y_stride; or y_splits partial sums of a product, y_split_stride elements
// apart, added up here) with mix [S, S] (from, to) and w_out [S]: update the streams.
// w_in [S] with norm_w [d]: h_out [n, d] = layer norm(sum_s w_in[s] xs[s]) * norm_w.  norm_w null: u_out float32 [n, d]
// = sum_s w_in[s] xs[s] (w_in null: the plain sum).  rows (or null): the tokens to work on, n of them.
int infero_hyper_step(float* xs, const float* y, int y_stride, int y_splits, long long y_split_stride, const float* mix,
                      const float* w_out, const float* w_in,
                      const float* norm_w, float eps, void* h_out, int h_dtype, float* u_out, const int* rows, int n,
                      int S, int d, cudaStream_t stream) {
    if (n == 0) return 0;
    const size_t sh = (size_t)d * sizeof(float);
    INFERO_REQUIRE(S >= 1 && S <= MAX_STREAMS, "hyper-connections: %d streams outside 1..%d", S, MAX_STREAMS);
    INFERO_REQUIRE(d >= 1 && sh <= 48 * 1024, "hyper-connections: width %d outside 1..12288", d);
    INFERO_REQUIRE(!y || (mix && w_out && y_splits >= 1), "hyper-connections: an update needs its mix matrix and output weights");
    INFERO_REQUIRE(!norm_w || h_out, "hyper-connections: a norm needs somewhere to write");
    const int threads = n <= 64 && d > THREADS ? THREADS_FEW : THREADS;
    if (h_dtype == INFERO_F32)
        hyper_step_kernel<float><<<n, threads, sh, stream>>>(xs, y, y_stride, y_splits, y_split_stride, mix, w_out, w_in, norm_w, eps,
                                                           (float*)h_out,
                                                           u_out, rows, S, d);
    else
        hyper_step_kernel<bf16><<<n, threads, sh, stream>>>(xs, y, y_stride, y_splits, y_split_stride, mix, w_out, w_in, norm_w, eps,
                                                          (bf16*)h_out,
                                                          u_out, rows, S, d);
    return infero_check_launch("hyper_step");
}

int infero_streams_fill(const float* x, float* xs, int n, int S, int d, cudaStream_t stream) {
    if (n == 0) return 0;
    streams_fill_kernel<<<n, THREADS, 0, stream>>>(x, xs, S, d);
    return infero_check_launch("streams_fill");
}

}  // extern "C"

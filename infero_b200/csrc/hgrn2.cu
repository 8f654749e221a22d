// HGRN2: gated linear recurrence with a matrix state per head, in which the forget gate also
// decides what is written.  Per head, with q_t (D), f_t in (0,1)^D and v_t (V):
//
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T        S is D x V, 32-bit, one per request and head
//   o_t = S_t^T q_t                                  then o_t / sqrt(mean(o_t^2) + eps) * w  over V
//
// q_t = silu(q'_t), f_t = l + (1 - l) sigmoid(f'_t + b) with q', f', v rows of one stacked product.
// One block per (head, request of the step) walks that request's new tokens in order, from the state
// the steps before left in the request's slot, and leaves the state behind; a step of one token is
// the same walk of length one.  Thread (j, s) keeps rows s*DPT .. s*DPT+DPT-1 of column j of S in
// registers; tokens are staged eight at a time in shared memory with the activations applied once.
//
// A long portion (LONG tokens and more) is cut into chunks of CHUNK tokens that run side by side, in three
// launches, because the recurrence is linear in S: (1) every chunk walks its tokens from a zero state and keeps
// its end state L_c and the product P_c of its forget gates; (2) one block per (head, request) strings them
// together, S_(c+1) = diag(P_c) S_c + L_c from the request's state, leaving every chunk's start state where L_c
// was; (3) every chunk walks its tokens again from its start state and writes the results.  Whether a request
// goes that way depends on its own portion alone, so what is computed for it does not depend on the batch.
#include "common.cuh"

namespace {

constexpr int TT = 8;      // tokens staged per round
constexpr int CHUNK = 128, LONG = 512;
enum { WHOLE = 0, LOCAL = 1, FROM_START = 2 };

template <typename T, int DPT, int MODE>
__global__ void __launch_bounds__(512, DPT <= 16 ? 2 : 1)          // (64 rows per thread: wide states, slow but whole)
hgrn2_scan_kernel(const float* __restrict__ proj, int stride, int q_off, int f_off, int v_off,
                  const float* __restrict__ f_bias, const float* __restrict__ lower,
                  const float* __restrict__ out_w, float eps, float* __restrict__ state,
                  const int* __restrict__ entry_q_start, const int* __restrict__ entry_q_len,
                  const int* __restrict__ entry_slot, T* __restrict__ out, int out_stride,
                  int H, int D, int V, int DS, float* __restrict__ chunk_state, float* __restrict__ chunk_decay,
                  const int* __restrict__ entry_chunk0, int long_from) {
    constexpr int mode = MODE;
    extern __shared__ __align__(16) float sm[];
    float* qs = sm;                      // [TT][D]
    float* fs = qs + TT * D;             // [TT][D]
    float* gs = fs + TT * D;             // [TT][D]: 1 - f
    float* vs = gs + TT * D;             // [TT][V]
    float* part = vs + TT * V;           // [TT][DS][V]
    const int h = blockIdx.x, e = blockIdx.y;
    int row0 = entry_q_start[e], n = entry_q_len[e];
    const int slot = entry_slot[e];
    const bool is_long = n >= long_from;                    // (without scratch for chunks every portion runs whole)
    if ((mode == WHOLE) == is_long) return;                 // long portions go by chunks, the others whole
    float* st_chunk = nullptr;
    float* decay = nullptr;
    if (mode != WHOLE) {
        const int c = blockIdx.z;
        if (c * CHUNK >= n) return;
        const size_t ci = (size_t)entry_chunk0[e] + c;
        st_chunk = chunk_state + (ci * H + blockIdx.x) * D * V;
        decay = chunk_decay + (ci * H + blockIdx.x) * D;
        row0 += c * CHUNK;
        n = min(CHUNK, n - c * CHUNK);
    }
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int j = tid % V, s = tid / V;
    const bool active = s < DS;
    const int i0 = s * DPT;
    float S[DPT];
    float* st = mode == WHOLE ? state + (((size_t)slot * H + h) * D) * V : st_chunk;
#pragma unroll
    for (int ii = 0; ii < DPT; ++ii) S[ii] = (mode != LOCAL && active && i0 + ii < D) ? st[(size_t)(i0 + ii) * V + j] : 0.f;
    float* pd = part + TT * DS * V;                          // [D]: product of the forget gates (LOCAL)
    for (int i = tid; i < D; i += nthreads) pd[i] = 1.f;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    for (int t0 = 0; t0 < n; t0 += TT) {
        const int nt = min(TT, n - t0);
        __syncthreads();
        for (int idx = tid; idx < nt * D; idx += nthreads) {
            const int tt = idx / D, i = idx - tt * D;
            const float* pr = proj + (size_t)(row0 + t0 + tt) * stride;
            if (mode != LOCAL) {
                const float qv = pr[q_off + h * D + i];
                qs[tt * D + i] = qv / (1.0f + expf(-qv));
            }
            const float fr = pr[f_off + h * D + i] + f_bias[h * D + i];
            const float l = lower[h * D + i];
            const float f = l + (1.0f - l) * (1.0f / (1.0f + expf(-fr)));
            fs[tt * D + i] = f;
            gs[tt * D + i] = 1.0f - f;
        }
        for (int idx = tid; idx < nt * V; idx += nthreads) {
            const int tt = idx / V, jj = idx - tt * V;
            vs[tt * V + jj] = proj[(size_t)(row0 + t0 + tt) * stride + v_off + h * V + jj];
        }
        __syncthreads();
        if (active) {
            const bool vec = (D & 3) == 0 && i0 + DPT <= D;      // this thread's channels as 16-byte reads (all lanes alike)
            // one token: S <- f S + g v_j (g = 1 - f), and, unless only the end state is wanted, o_j += S q
            auto token = [&](int tt) {
                const float vj = vs[tt * V + j];
                float o = 0.f;
                if (vec) {
                    const float4* f4 = reinterpret_cast<const float4*>(fs + tt * D + i0);
                    const float4* g4 = reinterpret_cast<const float4*>(gs + tt * D + i0);
                    const float4* q4 = reinterpret_cast<const float4*>(qs + tt * D + i0);
#pragma unroll
                    for (int k = 0; k < DPT / 4; ++k) {
                        const float4 f = f4[k], g = g4[k];
                        S[4 * k] = fmaf(f.x, S[4 * k], g.x * vj);
                        S[4 * k + 1] = fmaf(f.y, S[4 * k + 1], g.y * vj);
                        S[4 * k + 2] = fmaf(f.z, S[4 * k + 2], g.z * vj);
                        S[4 * k + 3] = fmaf(f.w, S[4 * k + 3], g.w * vj);
                        if (mode != LOCAL) {
                            const float4 q = q4[k];
                            o = fmaf(S[4 * k], q.x, o), o = fmaf(S[4 * k + 1], q.y, o);
                            o = fmaf(S[4 * k + 2], q.z, o), o = fmaf(S[4 * k + 3], q.w, o);
                        }
                    }
                } else {
#pragma unroll
                    for (int ii = 0; ii < DPT; ++ii) {
                        if (i0 + ii < D) {
                            S[ii] = fmaf(fs[tt * D + i0 + ii], S[ii], gs[tt * D + i0 + ii] * vj);
                            o = fmaf(S[ii], qs[tt * D + i0 + ii], o);
                        }
                    }
                }
                if (mode != LOCAL) part[(tt * DS + s) * V + j] = o;
            };
#pragma unroll 1
            for (int tt = 0; tt < nt; ++tt) token(tt);
        }
        if (mode == LOCAL) {                                 // (channel i stays with the same thread in every round)
            for (int i = tid; i < D; i += nthreads) {
                float p = pd[i];
                for (int tt = 0; tt < nt; ++tt) p *= fs[tt * D + i];
                pd[i] = p;
            }
        }
        __syncthreads();
        if (mode == LOCAL) continue;                         // only the end state is wanted
        for (int tt = warp; tt < nt; tt += nwarps) {
            float ss = 0.f;
            for (int jj = lane; jj < V; jj += 32) {
                float o = 0.f;
                for (int k = 0; k < DS; ++k) o += part[(tt * DS + k) * V + jj];
                part[(tt * DS) * V + jj] = o;
                ss = fmaf(o, o, ss);
            }
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)V + eps);
            T* orow = out + (size_t)(row0 + t0 + tt) * out_stride + (size_t)h * V;
            for (int jj = lane; jj < V; jj += 32) orow[jj] = from_f32<T>(part[(tt * DS) * V + jj] * r * out_w[jj]);
        }
    }
    if (active && mode != FROM_START) {
#pragma unroll
        for (int ii = 0; ii < DPT; ++ii)
            if (i0 + ii < D) {
                st[(size_t)(i0 + ii) * V + j] = S[ii];
            }
    }
    if (mode == LOCAL) {
        for (int i = tid; i < D; i += nthreads) decay[i] = pd[i];
    }
}

// S_(c+1) = diag(P_c) S_c + L_c over the chunks of every long portion; chunk_state[c] becomes S_c.  One thread per
// element of the state; the chunks' values are fetched eight at a time before the chain runs over them.
__global__ void hgrn2_chain_kernel(float* __restrict__ state, float* __restrict__ chunk_state,
                                   const float* __restrict__ chunk_decay, const int* __restrict__ entry_q_len,
                                   const int* __restrict__ entry_slot, const int* __restrict__ entry_chunk0,
                                   int H, int D, int V) {
    const int h = blockIdx.x, e = blockIdx.y;
    const int n = entry_q_len[e];
    if (n < LONG) return;
    const int idx = blockIdx.z * blockDim.x + threadIdx.x;
    if (idx >= D * V) return;
    const int chunks = (n + CHUNK - 1) / CHUNK;
    const int i = idx / V;
    float* st = state + (((size_t)entry_slot[e] * H + h) * D) * V;
    float S = st[idx];
    const size_t c_first = (size_t)entry_chunk0[e];
    for (int c0 = 0; c0 < chunks; c0 += 8) {
        float l[8], p[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < chunks) {
                l[k] = chunk_state[((c_first + c0 + k) * H + h) * D * V + idx];
                p[k] = chunk_decay[((c_first + c0 + k) * H + h) * D + i];
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < chunks) {
                chunk_state[((c_first + c0 + k) * H + h) * D * V + idx] = S;
                S = fmaf(p[k], S, l[k]);
            }
        }
    }
    st[idx] = S;
}

template <typename T, int DPT>
int launch(const float* proj, int stride, int q_off, int f_off, int v_off, const float* f_bias, const float* lower,
           const float* out_w, float eps, float* state, const int* qs, const int* ql, const int* es, void* out,
           int out_stride, int E, int H, int D, int V, int max_chunks, float* chunk_state, float* chunk_decay,
           const int* entry_chunk0, int any_short, cudaStream_t stream) {
    const int DS = (D + DPT - 1) / DPT;
    const int threads = ((V * DS + 31) / 32) * 32;
    const size_t smem = ((size_t)TT * (3 * D + V + DS * V) + D) * sizeof(float);
    auto kern = hgrn2_scan_kernel<T, DPT, WHOLE>;
    auto kern_local = hgrn2_scan_kernel<T, DPT, LOCAL>;
    auto kern_from = hgrn2_scan_kernel<T, DPT, FROM_START>;
    if (smem > 48 * 1024) {
        INFERO_REQUIRE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
                       cudaFuncSetAttribute(kern_local, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
                       cudaFuncSetAttribute(kern_from, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess,
                       "hgrn2: %zu bytes of shared memory are not available", smem);
    }
    if (any_short)
        kern<<<dim3(H, E), threads, smem, stream>>>(proj, stride, q_off, f_off, v_off, f_bias, lower, out_w, eps, state,
                                                    qs, ql, es, (T*)out, out_stride, H, D, V, DS, nullptr, nullptr, nullptr,
                                                    max_chunks > 0 ? LONG : 0x7fffffff);
    if (max_chunks > 0) {
        kern_local<<<dim3(H, E, max_chunks), threads, smem, stream>>>(proj, stride, q_off, f_off, v_off, f_bias, lower, out_w, eps,
            state, qs, ql, es, (T*)out, out_stride, H, D, V, DS, chunk_state, chunk_decay, entry_chunk0, LONG);
        hgrn2_chain_kernel<<<dim3(H, E, (D * V + 255) / 256), 256, 0, stream>>>(state, chunk_state, chunk_decay, ql, es, entry_chunk0, H, D, V);
        kern_from<<<dim3(H, E, max_chunks), threads, smem, stream>>>(proj, stride, q_off, f_off, v_off, f_bias, lower, out_w, eps,
            state, qs, ql, es, (T*)out, out_stride, H, D, V, DS, chunk_state, chunk_decay, entry_chunk0, LONG);
    }
    return infero_check_launch("hgrn2_scan");
}

}  // namespace

extern "C" {

int infero_hgrn2_chunk() { return CHUNK; }
int infero_hgrn2_long() { return LONG; }

// proj: float32 [tokens, stride] holding q' at column q_off (H*D), f' at f_off (H*D), v at v_off (H*V).
// state: float32 [slots, H, D, V].  out: [tokens, H*V] of out_dtype.
// Portions of infero_hgrn2_long() tokens and more run by chunks of infero_hgrn2_chunk(): max_chunks is the largest
// chunk count of any such portion (0: there is none), entry_chunk0[e] the first chunk index of entry e in
// chunk_state float32 [chunks, H, D, V] and chunk_decay float32 [chunks, H, D]; any_short: some portion is shorter.
int infero_hgrn2_scan(const float* proj, int stride, int q_off, int f_off, int v_off, const float* f_bias,
                      const float* lower, const float* out_w, float eps, float* state, const int* entry_q_start,
                      const int* entry_q_len, const int* entry_slot, void* out, int out_dtype, int out_stride,
                      int n_entries, int H, int D, int V, int max_chunks, float* chunk_state, float* chunk_decay,
                      const int* entry_chunk0, int any_short, cudaStream_t stream) {
    if (n_entries == 0) return 0;
    INFERO_REQUIRE(H > 0 && D > 0 && V > 0 && V <= 512, "hgrn2: bad sizes H=%d D=%d V=%d", H, D, V);
    int dpt = 8;
    while (dpt < 64 && V * ((D + dpt - 1) / dpt) > 512) dpt *= 2;
    INFERO_REQUIRE(V * ((D + dpt - 1) / dpt) <= 512, "hgrn2: a state of %d x %d per head is too large", D, V);
#define GO(TY, N) return launch<TY, N>(proj, stride, q_off, f_off, v_off, f_bias, lower, out_w, eps, state, \
                                       entry_q_start, entry_q_len, entry_slot, out, out_stride, n_entries, H, D, V, max_chunks, chunk_state, \
                                       chunk_decay, entry_chunk0, any_short, stream)
    if (out_dtype == INFERO_F32) {
        if (dpt == 8) GO(float, 8); if (dpt == 16) GO(float, 16); if (dpt == 32) GO(float, 32); GO(float, 64);
    } else {
        if (dpt == 8) GO(bf16, 8); if (dpt == 16) GO(bf16, 16); if (dpt == 32) GO(bf16, 32); GO(bf16, 64);
    }
#undef GO
}

}  // extern "C"

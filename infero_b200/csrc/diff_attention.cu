// Differential attention over the paged cache, and what runs in front of it.
//
// A head has two attention maps over the same values.  The stacked product of a token holds, head by
// head, query [map 1 | map 2] (each D wide), key [map 1 | map 2] per kv head and one value (V wide) per
// kv head.  The cache keeps a key row of width 2 D ([map 1 | map 2]) and a value row of width V.
//
// (1) qkv_prepare: a short causal convolution over time on every channel (taps values ending at the
//     token; what lies before this step's first token comes from the request's state slot, zeros before
//     the sequence's start), RMS norm of every map of every query and key head with a shared weight,
//     rotary positions on adjacent pairs (2i, 2i+1) of the first `rot` dimensions of each map, then the
//     query to its buffer and key and value to their pages.  One warp per token and map, 32-bit throughout.
// (2) conv_state_update: the last taps-1 raw product rows of every request become its new state.
// (3) diff_attention_generic: one warp per (token, head): two causal softmaxes (32-bit, running maximum
//     and sum, keys in ascending order in chunks of 32 aligned to absolute positions) a1, a2 over the
//     same values, o = a1 - lambda a2, o / sqrt(mean(o^2) + eps) * out_scale.  What is done for a token
//     depends only on its own position, never on the cut of the step or on the rest of the batch.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int PREP_WARPS = 8;
constexpr int MAX_TAPS = 16;
constexpr int SEG_MAX = 256;             // widest segment (one map of a head) a warp keeps in registers

// One warp per (token, segment).  The token's channels [q | k | v] are cut into segments of D: every map of every
// query and key head is one (normed and rotated), the values follow in pieces of D (copied).  Lane l holds channels
// l, l + 32, ... of its segment, so loads and stores are coalesced and the partner of a rotary pair sits in the
// neighbouring lane.
template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
qkv_prepare_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ conv_w, int taps,
                   const float* __restrict__ conv_state, const float* __restrict__ q_norm,
                   const float* __restrict__ k_norm, float eps, const float* __restrict__ inv_freq, int rot,
                   const int* __restrict__ positions, const int* __restrict__ tok_entry,
                   const int* __restrict__ entry_q_start, const int* __restrict__ entry_slot,
                   const int* __restrict__ block_table, int max_blocks, T* __restrict__ q_out, int q_stride,
                   T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int n_q_units, int n_k_units,
                   int G, int D, int V, int write_cache, int q_pad) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Cq = n_q_units * D, Ck = n_k_units * D, Cv = G * V, C = Cq + Ck + Cv;
    const int n_units = n_q_units + n_k_units, n_seg = n_units + (Cv + D - 1) / D;
    const int seg = blockIdx.y * PREP_WARPS + warp;
    const int t = blockIdx.x;
    const int pos = positions[t];
    __shared__ float2 cs_tab[SEG_MAX / 2];                     // (cos, sin) of the token's angles, shared by the block's maps
    if (blockIdx.y * PREP_WARPS < n_units) {                   // (a block of value segments only has no use for them)
        for (int i = threadIdx.x; i < rot / 2; i += PREP_WARPS * 32) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            cs_tab[i] = make_float2(cs, sn);
        }
        __syncthreads();
    }
    if (seg >= n_seg) return;
    const int e = tok_entry[t];
    const int r = t - entry_q_start[e];       // index of the token among its request's new tokens
    const int keep = taps - 1;
    const float* st = (taps > 1) ? conv_state + (size_t)entry_slot[e] * keep * C : nullptr;
    const int c0 = seg * D;                                   // first channel of the segment
    const int width = seg < n_units ? D : min(D, C - c0);

    float x[SEG_MAX / 32];
#pragma unroll
    for (int k = 0; k < SEG_MAX / 32; ++k) {
        const int i = k * 32 + lane;
        float acc = 0.f;
        if (i < width) {
            const int c = c0 + i;
            if (taps <= 0) {
                acc = proj[(size_t)t * stride + c];
            } else {
                for (int j = 0; j < taps; ++j) {
                    const int back = keep - j;                  // how many tokens before this one
                    const float u = (r - back >= 0) ? proj[(size_t)(t - back) * stride + c]
                                                    : st[(size_t)(r - back + keep) * C + c];
                    acc = fmaf(conv_w[(size_t)j * C + c], u, acc);
                }
            }
        }
        x[k] = acc;
    }
    if (seg < n_units) {
        const float* w = seg < n_q_units ? q_norm : k_norm;
        if (w) {
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < SEG_MAX / 32; ++k) ss = fmaf(x[k], x[k], ss);      // (channels beyond the width are 0)
            ss = warp_sum(ss);
            const float rn = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
            for (int k = 0; k < SEG_MAX / 32; ++k) {
                const int i = k * 32 + lane;
                if (i < D) x[k] = x[k] * rn * w[i];
            }
        }
#pragma unroll
        for (int k = 0; k < SEG_MAX / 32; ++k) {
            const int i = k * 32 + lane;                       // pair (2p, 2p + 1): the partner is the lane beside
            const float other = __shfl_xor_sync(0xffffffffu, x[k], 1);
            if (i < rot) {
                const float cs = cs_tab[i >> 1].x, sn = cs_tab[i >> 1].y;
                x[k] = (i & 1) ? x[k] * cs + other * sn : x[k] * cs - other * sn;
            }
        }
    }
    int page = -1;
    const int off = pos % page_size;
    if (seg >= n_q_units) {
        if (!write_cache) return;
        page = block_table[(size_t)e * max_blocks + pos / page_size];
        if (page < 0) return;
    }
    const int kw = G > 0 ? Ck / G : 0;                         // width of a key row: all maps of one kv head
#pragma unroll
    for (int k = 0; k < SEG_MAX / 32; ++k) {
        const int i = k * 32 + lane;
        if (i >= width) continue;
        const int c = c0 + i;
        if (seg < n_q_units) {
            if (q_pad) {
                // every map as a query of its own, as wide as a whole key row, with zeros where the other map's
                // columns are: unit u = 2 head + map goes to columns [2 D u + D map, + D)
                const int m = seg & 1;
                T* dst = q_out + (size_t)t * q_stride + (size_t)seg * 2 * D;
                dst[m * D + i] = from_f32<T>(x[k]);
                dst[(1 - m) * D + i] = from_f32<T>(0.f);
            } else {
                q_out[(size_t)t * q_stride + c] = from_f32<T>(x[k]);
            }
        } else if (seg < n_units) {
            const int ck = c - Cq, g = ck / kw, ii = ck - g * kw;
            k_cache[(((size_t)page * G + g) * page_size + off) * kw + ii] = from_f32<T>(x[k]);
        } else {
            const int cv = c - Cq - Ck, g = cv / V, ii = cv - g * V;
            v_cache[(((size_t)page * G + g) * page_size + off) * V + ii] = from_f32<T>(x[k]);
        }
    }
}

__global__ void conv_state_update_kernel(const float* __restrict__ proj, int stride, float* __restrict__ conv_state,
                                         int taps, const int* __restrict__ entry_q_start,
                                         const int* __restrict__ entry_q_len, const int* __restrict__ entry_slot,
                                         int C) {
    const int e = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int keep = taps - 1, n = entry_q_len[e], row0 = entry_q_start[e];
    float* st = conv_state + (size_t)entry_slot[e] * keep * C;
    float nv[MAX_TAPS];
#pragma unroll
    for (int s = 0; s < MAX_TAPS; ++s) {
        if (s < keep) {
            const int src = s + n;            // index in [old state (keep rows) | this step's rows]
            nv[s] = src < keep ? st[(size_t)src * C + c] : proj[(size_t)(row0 + src - keep) * stride + c];
        }
    }
#pragma unroll
    for (int s = 0; s < MAX_TAPS; ++s)
        if (s < keep) st[(size_t)s * C + c] = nv[s];
}

constexpr int WARPS = 4;
constexpr int MAX_D = 256;     // width of one map
constexpr int MAX_V = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
diff_attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                              const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                              const int* __restrict__ block_table, int max_blocks,
                              const int* __restrict__ tok_entry, const int* __restrict__ positions,
                              int n_tokens, int H, int G, int D, int V, int page_size, int window, float scale,
                              float lambda, float eps, float out_scale) {
    __shared__ float q_s[WARPS][2 * MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int g = h / (H / G);
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_entry[t] * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * 2 * D;
    for (int i = lane; i < 2 * D; i += 32) q_s[warp][i] = to_f32(qrow[i]);
    __syncwarp();

    float m1 = -CUDART_INF_F, l1 = 0.f, m2 = -CUDART_INF_F, l2 = 0.f;
    float acc1[MAX_V / 32], acc2[MAX_V / 32];
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) acc1[i] = acc2[i] = 0.f;

    for (int j0 = (lo / 32) * 32; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        long long row = -1;
        float s1 = -CUDART_INF_F, s2 = -CUDART_INF_F;
        if (j >= lo && j <= pos) {
            const int page = table[j / page_size];
            if (page >= 0) {
                row = ((long long)page * G + g) * page_size + (j % page_size);
                const T* kr = k_cache + row * 2 * D;
                float d1 = 0.f, d2 = 0.f;
                for (int i = 0; i < D; ++i) d1 = fmaf(q_s[warp][i], to_f32(kr[i]), d1);
                for (int i = 0; i < D; ++i) d2 = fmaf(q_s[warp][D + i], to_f32(kr[D + i]), d2);
                s1 = d1 * scale, s2 = d2 * scale;
            }
        }
        const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
        if (n1 == -CUDART_INF_F) continue;             // no readable key in this chunk (both maps see the same keys)
        const float p1 = (row >= 0) ? expf(s1 - n1) : 0.f, p2 = (row >= 0) ? expf(s2 - n2) : 0.f;
        const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
        l1 = l1 * c1 + warp_sum(p1);
        l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
        for (int i = 0; i < MAX_V / 32; ++i) acc1[i] *= c1, acc2[i] *= c2;
        for (int jj = 0; jj < 32; ++jj) {
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            const float pa = __shfl_sync(0xffffffffu, p1, jj), pb = __shfl_sync(0xffffffffu, p2, jj);
            if (rj < 0) continue;
            const T* vr = v_cache + rj * V;
#pragma unroll
            for (int i = 0; i < MAX_V / 32; ++i) {
                const int dd = i * 32 + lane;
                if (dd < V) {
                    const float v = to_f32(vr[dd]);
                    acc1[i] = fmaf(pa, v, acc1[i]);
                    acc2[i] = fmaf(pb, v, acc2[i]);
                }
            }
        }
        m1 = n1, m2 = n2;
    }
    const float i1 = 1.0f / l1, i2 = lambda / l2;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) {
        const int dd = i * 32 + lane;
        acc1[i] = dd < V ? acc1[i] * i1 - acc2[i] * i2 : 0.f;
        ss = fmaf(acc1[i], acc1[i], ss);
    }
    ss = warp_sum(ss);
    const float r = out_scale / sqrtf(ss / (float)V + eps);
    T* orow = out + (size_t)t * out_stride + (size_t)h * V;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) {
        const int dd = i * 32 + lane;
        if (dd < V) orow[dd] = from_f32<T>(acc1[i] * r);
    }
}

// maps [tokens, H, 2, V] (each map's attention result) -> out [tokens, H, V]: a1 - lambda a2, divided by its root
// mean square over V (plus eps), times out_scale.  One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
diff_combine_kernel(const T* __restrict__ maps, int maps_stride, T* __restrict__ out, int out_stride, int n_tokens, int H,
                    int V, float lambda, float eps, float out_scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const T* a1 = maps + (size_t)t * maps_stride + (size_t)h * 2 * V;
    const T* a2 = a1 + V;
    float o[MAX_V / 32];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) {
        const int dd = i * 32 + lane;
        o[i] = dd < V ? to_f32(a1[dd]) - lambda * to_f32(a2[dd]) : 0.f;
        ss = fmaf(o[i], o[i], ss);
    }
    ss = warp_sum(ss);
    const float r = out_scale / sqrtf(ss / (float)V + eps);
    T* orow = out + (size_t)t * out_stride + (size_t)h * V;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) {
        const int dd = i * 32 + lane;
        if (dd < V) orow[dd] = from_f32<T>(o[i] * r);
    }
}

}  // namespace

extern "C" {

int infero_diff_combine(const void* maps, int maps_stride, void* out, int out_stride, int dtype, int n_tokens, int H, int V,
                        float lambda, float eps, float out_scale, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(V >= 1 && V <= MAX_V, "diff combine: value width %d outside 1..%d", V, MAX_V);
    const unsigned blocks = (unsigned)(((long long)n_tokens * H + WARPS - 1) / WARPS);
    if (dtype == INFERO_F32)
        diff_combine_kernel<float><<<blocks, WARPS * 32, 0, stream>>>((const float*)maps, maps_stride, (float*)out, out_stride,
                                                                      n_tokens, H, V, lambda, eps, out_scale);
    else
        diff_combine_kernel<bf16><<<blocks, WARPS * 32, 0, stream>>>((const bf16*)maps, maps_stride, (bf16*)out, out_stride,
                                                                     n_tokens, H, V, lambda, eps, out_scale);
    return infero_check_launch("diff_combine");
}


// proj float32 [tokens, stride]: columns [q (n_q_units*D) | k (n_k_units*D) | v (G*V)] in front.
// conv_w float32 [taps, C] (tap j of channel c at j * C + c; the channels in that order); conv_state float32
// [slots, taps-1, C].
// taps 0: no convolution.  q_norm / k_norm float32 [D] or null.  inv_freq float32 [rot/2] (rot 0: none).
int infero_qkv_prepare(const float* proj, int stride, const float* conv_w, int taps, const float* conv_state,
                       const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rot,
                       const int* positions, const int* tok_entry, const int* entry_q_start, const int* entry_slot,
                       const int* block_table, int max_blocks, void* q_out, int q_stride, void* k_cache, void* v_cache,
                       int dtype, int page_size, int n_tokens, int n_q_units, int n_k_units, int G, int D, int V,
                       int write_cache, int q_pad, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(taps <= MAX_TAPS, "qkv_prepare: %d taps, at most %d", taps, MAX_TAPS);
    INFERO_REQUIRE(G > 0 && n_k_units % G == 0 && rot % 2 == 0 && rot <= D, "qkv_prepare: bad sizes");
    INFERO_REQUIRE(D >= 1 && D <= SEG_MAX, "qkv_prepare: map width %d outside 1..%d", D, SEG_MAX);
    const int n_seg = n_q_units + n_k_units + (G * V + D - 1) / D;
    INFERO_REQUIRE(n_seg <= 65535 * PREP_WARPS, "qkv_prepare: %d maps are too many", n_seg);
    const dim3 grid(n_tokens, (n_seg + PREP_WARPS - 1) / PREP_WARPS);
    if (dtype == INFERO_F32)
        qkv_prepare_kernel<float><<<grid, PREP_WARPS * 32, 0, stream>>>(proj, stride, conv_w, taps, conv_state, q_norm, k_norm,
            eps, inv_freq, rot, positions, tok_entry, entry_q_start, entry_slot, block_table, max_blocks, (float*)q_out,
            q_stride, (float*)k_cache, (float*)v_cache, page_size, n_q_units, n_k_units, G, D, V, write_cache, q_pad);
    else
        qkv_prepare_kernel<bf16><<<grid, PREP_WARPS * 32, 0, stream>>>(proj, stride, conv_w, taps, conv_state, q_norm, k_norm,
            eps, inv_freq, rot, positions, tok_entry, entry_q_start, entry_slot, block_table, max_blocks, (bf16*)q_out,
            q_stride, (bf16*)k_cache, (bf16*)v_cache, page_size, n_q_units, n_k_units, G, D, V, write_cache, q_pad);
    return infero_check_launch("qkv_prepare");
}

int infero_conv_state_update(const float* proj, int stride, float* conv_state, int taps, const int* entry_q_start,
                             const int* entry_q_len, const int* entry_slot, int n_entries, int C,
                             cudaStream_t stream) {
    if (n_entries == 0 || taps <= 1) return 0;
    INFERO_REQUIRE(taps <= MAX_TAPS, "conv_state_update: %d taps, at most %d", taps, MAX_TAPS);
    conv_state_update_kernel<<<dim3((C + 127) / 128, n_entries), 128, 0, stream>>>(proj, stride, conv_state, taps,
        entry_q_start, entry_q_len, entry_slot, C);
    return infero_check_launch("conv_state_update");
}

int infero_diff_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                                  const void* v_cache, int dtype, const int* block_table, int max_blocks,
                                  const int* tok_entry, const int* positions, int n_tokens, int H, int G, int D, int V,
                                  int page_size, int window, float scale, float lambda, float eps, float out_scale,
                                  cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(D >= 1 && D <= MAX_D && V >= 1 && V <= MAX_V, "diff attention: map width %d / value width %d outside 1..%d", D, V, MAX_D);
    INFERO_REQUIRE(G > 0 && H % G == 0, "diff attention: %d heads not a multiple of %d kv heads", H, G);
    const long long items = (long long)n_tokens * H;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (dtype == INFERO_F32)
        diff_attention_generic_kernel<float><<<blocks, WARPS * 32, 0, stream>>>((const float*)q, q_stride, (float*)out,
            out_stride, (const float*)k_cache, (const float*)v_cache, block_table, max_blocks, tok_entry, positions,
            n_tokens, H, G, D, V, page_size, window, scale, lambda, eps, out_scale);
    else
        diff_attention_generic_kernel<bf16><<<blocks, WARPS * 32, 0, stream>>>((const bf16*)q, q_stride, (bf16*)out,
            out_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, tok_entry, positions,
            n_tokens, H, G, D, V, page_size, window, scale, lambda, eps, out_scale);
    return infero_check_launch("diff_attention_generic");
}

}  // extern "C"

// Differential attention of bf16 steps: prompt portions on the warp-level tensor cores, single tokens on
// a block of warps that share a token's keys.
//
// diff_attn_prefill<D, V>: one CTA = 64 consecutive query tokens of one request and one head, eight warps:
//   warps 0-3 run map 1 and warps 4-7 map 2 of the same 64 rows (16 rows each), over the same tiles of 64
//   cached positions (a key row [map 1 | map 2] of width 2 D and a value row of width V per position),
//   gathered page by page with cp.async in two stages.  Scores, running maximum and sum are 32-bit, the
//   probabilities are rounded to bf16 for the second product.  At the end map 2's normalised result goes
//   through shared memory to the warps of map 1, which form a1 - lambda a2, divide by the root mean square
//   over V (plus eps) and scale.
// diff_attn_decode: one CTA = one token and one head; eight warps take the 32-key chunks of the context in
//   turn (chunk n to warp n mod 8, chunks aligned to absolute positions), each with both maps' running
//   statistics, and are merged in shared memory in warp order.  Also the 32-bit path's kernel for single
//   tokens (any element type).
#include "attn_common.cuh"

namespace {

using namespace attn;

constexpr int PF_ROWS = 64, PF_KEYS = 64, PF_THREADS = 256;

template <int D, int V>
__global__ void __launch_bounds__(PF_THREADS)
diff_attn_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                         const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                         const int* __restrict__ block_table, int max_blocks, const int* __restrict__ entry_q_start,
                         const int* __restrict__ entry_q_len, const int* __restrict__ entry_pos0, int n_entries,
                         int first_entry, int H, int G, int page_size, int window, float scale_log2, float lambda,
                         float eps, float out_scale) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* tiles = reinterpret_cast<bf16*>(smem_raw);          // [2 stages][K 64 x 2D | V 64 x V]
    constexpr int KT = tile_elems<2 * D>(PF_KEYS), VT = tile_elems<V>(PF_KEYS), STAGE = KT + VT;

    int e = -1, tile_in_e = 0;
    {
        int left = blockIdx.x;
        for (int i = first_entry; i < n_entries; ++i) {
            const int nt = (entry_q_len[i] + PF_ROWS - 1) / PF_ROWS;
            if (left < nt) { e = i; tile_in_e = left; break; }
            left -= nt;
        }
    }
    if (e < 0) return;
    const int h = blockIdx.y, kvh = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int map = warp >> 2, w4 = warp & 3;
    const int q_len = entry_q_len[e], pos0 = entry_pos0[e], tok0 = entry_q_start[e];
    const int* table = block_table + (size_t)e * max_blocks;
    const int row_first = tile_in_e * PF_ROWS;
    const int rows_here = min(PF_ROWS, q_len - row_first);
    const int wrow = row_first + w4 * 16;
    const int wvalid = max(0, min(16, q_len - wrow));

    uint32_t qf[D / 16][4];
    load_q<D>(qf, q + (size_t)(tok0 + wrow) * q_stride + (size_t)h * 2 * D + (size_t)map * D, (size_t)q_stride, wvalid, lane);

    const int p0 = pos0 + wrow + g, p1 = p0 + 8;
    const int hi0 = (g < wvalid) ? p0 : -1, hi1 = (g + 8 < wvalid) ? p1 : -1;
    const int lo0 = window > 0 ? max(0, p0 - window + 1) : 0, lo1 = window > 0 ? max(0, p1 - window + 1) : 0;
    const int cta_hi = pos0 + row_first + rows_here - 1;
    const int cta_lo = window > 0 ? max(0, pos0 + row_first - window + 1) : 0;
    const int key_begin = (cta_lo / PF_KEYS) * PF_KEYS;
    const int n_tiles = (cta_hi - key_begin) / PF_KEYS + 1;
    const int warp_hi = pos0 + wrow + wvalid - 1;
    const int warp_lo = window > 0 ? max(0, pos0 + wrow - window + 1) : 0;

    float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
    float o[V / 8][4];
#pragma unroll
    for (int i = 0; i < V / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    auto issue = [&](int t) {
        bf16* kt = tiles + (size_t)(t & 1) * STAGE;
        const int key0 = key_begin + t * PF_KEYS;
        gather_rows<2 * D>(kt, k_cache, table, key0, PF_KEYS, cta_hi + 1, G, kvh, page_size, threadIdx.x, PF_THREADS);
        gather_rows<V>(kt + KT, v_cache, table, key0, PF_KEYS, cta_hi + 1, G, kvh, page_size, threadIdx.x, PF_THREADS);
        cp_async_commit();
    };
    issue(0);
    for (int t = 0; t < n_tiles; ++t) {
        if (t + 1 < n_tiles) issue(t + 1);
        else cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* kt = tiles + (size_t)(t & 1) * STAGE;
        const int key0 = key_begin + t * PF_KEYS;
        if (wvalid > 0 && key0 <= warp_hi && key0 + PF_KEYS > warp_lo) {
#pragma unroll 1
            for (int sl = 0; sl < PF_KEYS / KEYS16; ++sl) {
                const int kb = key0 + sl * KEYS16;
                if (kb > warp_hi || kb + KEYS16 <= warp_lo) continue;
                slice16_kv<D, V, PaddedRows<2 * D>, PaddedRows<V>>(qf, kt, kt + KT, sl * KEYS16, kb, lo0, hi0, lo1, hi1,
                                                                     scale_log2, m, l, o, lane, map * (D / 8));
            }
        }
        __syncthreads();
    }
    float l0 = l[0], l1 = l[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
    // map 2 hands its normalised rows to map 1 (the tiles are no longer read: the loop ended on a barrier)
    float* xch = reinterpret_cast<float*>(smem_raw);                   // [64][V]
    float* x0 = xch + (size_t)(w4 * 16 + g) * V;
    float* x1 = x0 + (size_t)8 * V;
    if (map == 1) {
#pragma unroll
        for (int nt = 0; nt < V / 8; ++nt) {
            const int d = nt * 8 + c * 2;
            *reinterpret_cast<float2*>(x0 + d) = make_float2(o[nt][0] * inv0, o[nt][1] * inv0);
            *reinterpret_cast<float2*>(x1 + d) = make_float2(o[nt][2] * inv1, o[nt][3] * inv1);
        }
    }
    __syncthreads();
    if (map == 0) {
        float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < V / 8; ++nt) {
            const int d = nt * 8 + c * 2;
            const float2 b0 = *reinterpret_cast<const float2*>(x0 + d), b1 = *reinterpret_cast<const float2*>(x1 + d);
            o[nt][0] = o[nt][0] * inv0 - lambda * b0.x;
            o[nt][1] = o[nt][1] * inv0 - lambda * b0.y;
            o[nt][2] = o[nt][2] * inv1 - lambda * b1.x;
            o[nt][3] = o[nt][3] * inv1 - lambda * b1.y;
            ss0 += o[nt][0] * o[nt][0] + o[nt][1] * o[nt][1];
            ss1 += o[nt][2] * o[nt][2] + o[nt][3] * o[nt][3];
        }
        ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
        ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
        ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
        ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
        const float r0 = out_scale / sqrtf(ss0 / (float)V + eps), r1 = out_scale / sqrtf(ss1 / (float)V + eps);
        bf16* orow0 = out + (size_t)(tok0 + wrow + g) * out_stride + (size_t)h * V;
        bf16* orow1 = orow0 + (size_t)8 * out_stride;
#pragma unroll
        for (int nt = 0; nt < V / 8; ++nt) {
            const int d = nt * 8 + c * 2;
            if (g < wvalid) *reinterpret_cast<uint32_t*>(orow0 + d) = pack_bf16(o[nt][0] * r0, o[nt][1] * r0);
            if (g + 8 < wvalid) *reinterpret_cast<uint32_t*>(orow1 + d) = pack_bf16(o[nt][2] * r1, o[nt][3] * r1);
        }
    }
}

template <int D, int V>
int launch_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_cache, const void* v_cache,
                   const int* block_table, int max_blocks, const int* entry_q_start, const int* entry_q_len,
                   const int* entry_pos0, int n_entries, int first_entry, int n_tiles, int H, int G, int page_size,
                   int window, float scale_log2, float lambda, float eps, float out_scale, cudaStream_t stream) {
    auto kern = diff_attn_prefill_kernel<D, V>;
    int smem = 2 * (tile_elems<2 * D>(PF_KEYS) + tile_elems<V>(PF_KEYS)) * 2;
    if (smem < PF_ROWS * V * 4) smem = PF_ROWS * V * 4;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    kern<<<dim3(n_tiles, H), PF_THREADS, smem, stream>>>((const bf16*)q, q_stride, (bf16*)out, out_stride,
        (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, entry_q_start, entry_q_len, entry_pos0,
        n_entries, first_entry, H, G, page_size, window, scale_log2, lambda, eps, out_scale);
    return infero_check_launch("diff_attn_prefill");
}

// ---- single tokens ------------------------------------------------------------------------------------------
constexpr int DW = 16;             // warps of a block
constexpr int MAX_D = 256, MAX_V = 256;

// q . k over n elements; bf16 rows whose length is a multiple of 8 are read 16 bytes at a time
__device__ __forceinline__ float dot_q(const float* __restrict__ q, const float* __restrict__ k, int n) {
    float d = 0.f;
    for (int i = 0; i < n; ++i) d = fmaf(q[i], k[i], d);
    return d;
}
__device__ __forceinline__ float dot_q(const float* __restrict__ q, const bf16* __restrict__ k, int n) {
    float d = 0.f;
    if ((n & 7) == 0 && ((uintptr_t)k & 15) == 0) {
        for (int i = 0; i < n; i += 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(k + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(p[j]);
                d = fmaf(q[i + 2 * j], f.x, d);
                d = fmaf(q[i + 2 * j + 1], f.y, d);
            }
        }
        return d;
    }
    for (int i = 0; i < n; ++i) d = fmaf(q[i], __bfloat162float(k[i]), d);
    return d;
}

// PAIR: a lane owns adjacent value columns (2 lane, 2 lane + 1) of every block of 64 (bf16 pairs, 4-byte loads);
// else column lane of every block of 32.
template <typename T, bool PAIR>
__global__ void __launch_bounds__(DW * 32)
diff_attn_decode_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                        const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_entry,
                        const int* __restrict__ positions, int H, int G, int D, int V, int page_size, int window,
                        float scale, float lambda, float eps, float out_scale) {
    extern __shared__ float sm[];
    float* q_s = sm;                         // [2 D]
    float* st = q_s + 2 * D;                 // [DW][4]: m1, l1, m2, l2
    float* accs = st + DW * 4;               // [DW][2][V]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, h = blockIdx.y;
    const int g = h / (H / G);
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_entry[t] * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * 2 * D;
    for (int i = threadIdx.x; i < 2 * D; i += DW * 32) q_s[i] = to_f32(qrow[i]);
    __syncthreads();

    float m1 = -CUDART_INF_F, l1 = 0.f, m2 = -CUDART_INF_F, l2 = 0.f;
    float acc1[MAX_V / 32], acc2[MAX_V / 32];
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) acc1[i] = acc2[i] = 0.f;
    const int first_chunk = lo / 32;
    for (int ch = first_chunk + ((warp - first_chunk) % DW + DW) % DW; ch * 32 <= pos; ch += DW) {   // chunk n belongs to warp n mod DW
        const int j = ch * 32 + lane;
        long long row = -1;
        float s1 = -CUDART_INF_F, s2 = -CUDART_INF_F;
        if (j >= lo && j <= pos) {
            const int page = table[j / page_size];
            if (page >= 0) {
                row = ((long long)page * G + g) * page_size + (j % page_size);
                const T* kr = k_cache + row * 2 * D;
                s1 = dot_q(q_s, kr, D) * scale, s2 = dot_q(q_s + D, kr + D, D) * scale;
            }
        }
        const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
        if (n1 == -CUDART_INF_F) continue;
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
            if (PAIR) {
#pragma unroll
                for (int i = 0; i < MAX_V / 64; ++i) {
                    const int dd = i * 64 + 2 * lane;
                    if (dd < V) {
                        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>((const bf16*)vr + dd));
                        acc1[2 * i] = fmaf(pa, v.x, acc1[2 * i]), acc1[2 * i + 1] = fmaf(pa, v.y, acc1[2 * i + 1]);
                        acc2[2 * i] = fmaf(pb, v.x, acc2[2 * i]), acc2[2 * i + 1] = fmaf(pb, v.y, acc2[2 * i + 1]);
                    }
                }
            } else {
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
        }
        m1 = n1, m2 = n2;
    }
    // the column register i of this lane holds
    auto col = [&](int i) { return PAIR ? (i >> 1) * 64 + 2 * lane + (i & 1) : i * 32 + lane; };
    if (lane == 0) st[warp * 4 + 0] = m1, st[warp * 4 + 1] = l1, st[warp * 4 + 2] = m2, st[warp * 4 + 3] = l2;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) {
        const int dd = col(i);
        if (dd < V) accs[(warp * 2 + 0) * V + dd] = acc1[i], accs[(warp * 2 + 1) * V + dd] = acc2[i];
    }
    __syncthreads();
    if (warp != 0) return;
    float M1 = -CUDART_INF_F, M2 = -CUDART_INF_F;
    for (int w = 0; w < DW; ++w) M1 = fmaxf(M1, st[w * 4]), M2 = fmaxf(M2, st[w * 4 + 2]);
    float L1 = 0.f, L2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) acc1[i] = acc2[i] = 0.f;
    for (int w = 0; w < DW; ++w) {
        const float f1 = st[w * 4] == -CUDART_INF_F ? 0.f : expf(st[w * 4] - M1);
        const float f2 = st[w * 4 + 2] == -CUDART_INF_F ? 0.f : expf(st[w * 4 + 2] - M2);
        L1 = fmaf(st[w * 4 + 1], f1, L1);
        L2 = fmaf(st[w * 4 + 3], f2, L2);
#pragma unroll
        for (int i = 0; i < MAX_V / 32; ++i) {
            const int dd = col(i);
            if (dd < V) {
                acc1[i] = fmaf(accs[(w * 2 + 0) * V + dd], f1, acc1[i]);
                acc2[i] = fmaf(accs[(w * 2 + 1) * V + dd], f2, acc2[i]);
            }
        }
    }
    const float i1 = 1.0f / L1, i2 = lambda / L2;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) {
        const int dd = col(i);
        acc1[i] = dd < V ? acc1[i] * i1 - acc2[i] * i2 : 0.f;
        ss = fmaf(acc1[i], acc1[i], ss);
    }
    ss = warp_sum(ss);
    const float r = out_scale / sqrtf(ss / (float)V + eps);
    T* orow = out + (size_t)t * out_stride + (size_t)h * V;
#pragma unroll
    for (int i = 0; i < MAX_V / 32; ++i) {
        const int dd = col(i);
        if (dd < V) orow[dd] = from_f32<T>(acc1[i] * r);
    }
}

bool prefill_sizes_ok(int D, int V) {
    auto ok = [](int n) { return n == 32 || n == 48 || n == 64 || n == 96 || n == 128; };
    return ok(D) && ok(V);
}

}  // namespace

extern "C" {

int infero_diff_attn_prefill_supported(int D, int V, int page_size) {
    return prefill_sizes_ok(D, V) && page_size % 16 == 0;
}

// Prompt portions (and whatever single tokens follow them) of entries first_entry..n_entries-1; n_tiles is the
// number of blocks of 64 query rows they make.  bf16 only.
int infero_diff_attn_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                             const void* v_cache, const int* block_table, int max_blocks, const int* entry_q_start,
                             const int* entry_q_len, const int* entry_pos0, int n_entries, int first_entry, int n_tiles,
                             int H, int G, int D, int V, int page_size, int window, float scale, float lambda, float eps,
                             float out_scale, cudaStream_t stream) {
    if (n_tiles == 0) return 0;
    INFERO_REQUIRE(infero_diff_attn_prefill_supported(D, V, page_size), "diff_attn_prefill: sizes %d / %d / page %d have no instance", D, V, page_size);
    INFERO_REQUIRE(G > 0 && H % G == 0 && H <= 65535 && q_stride % 8 == 0 && out_stride % 2 == 0, "diff_attn_prefill: bad head counts or strides");
    const float sl2 = scale * 1.4426950408889634f;
#define CALL(D_, V_) return launch_prefill<D_, V_>(q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_blocks, \
        entry_q_start, entry_q_len, entry_pos0, n_entries, first_entry, n_tiles, H, G, page_size, window, sl2, lambda, eps, out_scale, stream)
#define ROW(D_) if (D == D_) { if (V == 32) CALL(D_, 32); if (V == 48) CALL(D_, 48); if (V == 64) CALL(D_, 64); \
                               if (V == 96) CALL(D_, 96); CALL(D_, 128); }
    ROW(32) ROW(48) ROW(64) ROW(96) ROW(128)
#undef ROW
#undef CALL
    return 1;
}

// Tokens tok_first .. tok_first + n_tok - 1, each alone in its block of warps.
int infero_diff_attn_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                            const void* v_cache, int dtype, const int* block_table, int max_blocks, const int* tok_entry,
                            const int* positions, int n_tok, int H, int G, int D, int V, int page_size, int window,
                            float scale, float lambda, float eps, float out_scale, cudaStream_t stream) {
    if (n_tok == 0) return 0;
    INFERO_REQUIRE(D >= 1 && D <= MAX_D && V >= 1 && V <= MAX_V, "diff_attn_decode: map width %d / value width %d outside 1..%d", D, V, MAX_D);
    INFERO_REQUIRE(G > 0 && H % G == 0 && H <= 65535, "diff_attn_decode: %d heads / %d kv heads", H, G);
    const size_t smem = (size_t)(2 * D + DW * 4 + DW * 2 * V) * sizeof(float);
    const dim3 grid(n_tok, H);
    if (dtype == INFERO_F32)
        diff_attn_decode_kernel<float, false><<<grid, DW * 32, smem, stream>>>((const float*)q, q_stride, (float*)out, out_stride,
            (const float*)k_cache, (const float*)v_cache, block_table, max_blocks, tok_entry, positions, H, G, D, V,
            page_size, window, scale, lambda, eps, out_scale);
    else if (V % 2 == 0)
        diff_attn_decode_kernel<bf16, true><<<grid, DW * 32, smem, stream>>>((const bf16*)q, q_stride, (bf16*)out, out_stride,
            (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, tok_entry, positions, H, G, D, V,
            page_size, window, scale, lambda, eps, out_scale);
    else
        diff_attn_decode_kernel<bf16, false><<<grid, DW * 32, smem, stream>>>((const bf16*)q, q_stride, (bf16*)out, out_stride,
            (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, tok_entry, positions, H, G, D, V,
            page_size, window, scale, lambda, eps, out_scale);
    return infero_check_launch("diff_attn_decode");
}

}  // extern "C"

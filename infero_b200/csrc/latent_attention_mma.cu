// Latent attention on the warp-level tensor cores (bf16, mma.sync m16n8k16), for prompt portions and single tokens.
//
// All heads of a token read the same cached rows [c | rotated part] (width W = C + R), and a row's first C columns
// are also its value, so the heads are stacked as rows of one tile: a CTA works on ROWG * 16 rows = TQ tokens x HC
// heads of one request (HC = 16, 32 or 64 heads; TQ = 1 for single tokens, 64 / HC in a prompt portion) and walks
// the request's keys in tiles of 32, fetched once for all its rows by cp.async into a ring in shared memory.
// Queries arrive as float32 (the plain parts already carried through Wuk^T) and are rounded to bf16 into shared
// memory once; scores, running maximum and sum are 32-bit.  Two warps share 16 rows (four for single tokens with a
// latent of 256 and more, where a CTA has few rows and the length of a warp's instruction chain is what counts): each
// forms the rows' scores with its share of a tile's 32 keys, they exchange the rows' maxima and their softmax weights
// (as tensor-core fragments, whose layout is the same lane by lane) through shared memory, and each owns its share of the
// C result columns, so the result tile of 16 x C/2 (or C/4) stays in registers.  Key tiles start at multiples of 32 of the absolute position, so what is
// computed for a token does not depend on how its prompt was cut.
//
// Single tokens with long contexts are cut into `splits` ranges of keys, one CTA each; every CTA leaves its
// maximum, sum and unnormalised result, and a second kernel adds them up in ascending order.
#include "attn_common.cuh"

namespace {

using namespace attn;

constexpr int KT = 32;                        // keys per tile

// a barrier of the NW warps that share 16 rows (barrier 0 is the block's)
template <int NW>
__device__ __forceinline__ void group_sync(int rg) { asm volatile("bar.sync %0, %1;" ::"r"(rg + 1), "n"(NW * 32) : "memory"); }

// NW = 2 or 4 warps share 16 rows: each forms the scores of 32 / NW of a tile's keys and owns C / NW result columns.
template <int C, int ROWG, int STAGES, int NW>
__global__ void __launch_bounds__(ROWG * NW * 32, 1)
latent_mma_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, long long head_rows,
                  bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                  const bf16* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
                  const int* __restrict__ entry_q_start, const int* __restrict__ entry_q_len,
                  const int* __restrict__ entry_pos0, int entry_first, int n_entries, int TQ, int HC, int H, int R,
                  int page_size, float scale_log2, int chunk, int splits) {
    constexpr int ROWS = ROWG * 16, NT = ROWG * NW * 32, CW = C / NW, NO = CW / 8;
    constexpr int KW = KT / NW, NTW = KW / 8;              // keys, and n-tiles of 8 keys, whose scores a warp forms
    const int W = C + R, LD = W + 8;                       // padded row of a tile, in elements
    extern __shared__ __align__(16) uint8_t smem[];
    bf16* q_s = reinterpret_cast<bf16*>(smem);             // [ROWS][LD]
    bf16* k_s = q_s + ROWS * LD;                           // [STAGES][KT][LD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp / NW, part = warp % NW;
    // what the warps of 16 rows hand one another: their softmax weights as tensor-core fragments ([k-step of 16 keys][register]
    // [lane]: the fragment layout is the same in every warp, lane by lane), row maxima and, at the end, sums
    uint32_t* xp = reinterpret_cast<uint32_t*>(k_s + (size_t)STAGES * KT * LD) + rg * 256;    // [2][4][32]
    float* xm = reinterpret_cast<float*>(reinterpret_cast<uint32_t*>(k_s + (size_t)STAGES * KT * LD) + ROWG * 256) + rg * 64;   // [NW][16]

    // ---- which request, which of its tokens ---------------------------------------------------------------
    int e = entry_first, t0 = 0;
    if (TQ == 1 && ROWG < 4) {
        e = entry_first + blockIdx.x;                          // single tokens: a tile is a request
        if (e >= n_entries) return;
    } else {
        int tile = blockIdx.x;
        for (; e < n_entries; ++e) {
            const int n = (entry_q_len[e] + TQ - 1) / TQ;
            if (tile < n) break;
            tile -= n;
        }
        if (e >= n_entries) return;
        t0 = tile * TQ;
    }
    const int q_len = entry_q_len[e], tok0 = entry_q_start[e] + t0, pos_first = entry_pos0[e] + t0;
    const int n_tq = min(TQ, q_len - t0);
    const int head0 = blockIdx.y * HC;
    const int split = blockIdx.z;
    const int k_lo = split * chunk;
    const int k_hi = min(pos_first + n_tq, splits > 1 ? k_lo + chunk : 0x7fffffff);     // one past the last key
    const int* table = block_table + (size_t)e * max_blocks;

    // a tile row is fetched by NT / KT threads: its page was looked up while the tile before was being worked on
    // (`page_of` for the tile after is issued right behind the copies), then its 16-byte chunks go back to back
    constexpr int PER_ROW = NT / KT;
    const int lr = tid / PER_ROW, lc0 = tid % PER_ROW;
    auto page_of = [&](int key0) {
        const int j = key0 + lr;
        return (j >= k_lo && j < k_hi) ? table[j / page_size] : -1;
    };
    auto load_tile = [&](int stage, int key0, int page) {
        const int j = key0 + lr;
        bf16* d = k_s + ((size_t)stage * KT + lr) * LD;
        const int CH = W / 8;
        if (page >= 0) {
            const bf16* src = cache + ((size_t)page * page_size + (j % page_size)) * W;
            for (int c = lc0; c < CH; c += PER_ROW) cp_async16(smem_addr(d + c * 8), src + c * 8);
        } else {
            for (int c = lc0; c < CH; c += PER_ROW) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0, 0, 0, 0);
        }
    };
    const int key_begin = (k_lo / KT) * KT;
    const int n_tiles = k_hi > key_begin ? (k_hi - key_begin + KT - 1) / KT : 0;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_tiles) load_tile(s, key_begin + s * KT, page_of(key_begin + s * KT));
        cp_async_commit();
    }
    int page_next = STAGES - 1 < n_tiles ? page_of(key_begin + (STAGES - 1) * KT) : -1;
    // ---- queries: float32 -> bf16 rows [latent part | rotated part]; rows without a token or head are zero -------
    // (64 threads a row, four values per load, the loads of four rows in flight together; no division in the loop: with
    // two warps a CTA every instruction counts)
    {
        const int W4 = W / 4, C4 = C / 4;
        constexpr int RPI = NT / 64;                           // rows per pass
        const int sub = tid >> 6, c_first = tid & 63;
#pragma unroll 4
        for (int r = sub; r < ROWS; r += RPI) {
            const int tq = r / HC, n = head0 + r - tq * HC;
            const bool live = tq < n_tq && n < H;
            const size_t row = live ? (size_t)n * head_rows + tok0 + tq : 0;
            const float4* lat = reinterpret_cast<const float4*>(q_lat + row * C);
            const float4* rot = reinterpret_cast<const float4*>(q_rot + row * R) - C4;
            bf16* dst = q_s + (size_t)r * LD;
            for (int c = c_first; c < W4; c += 64) {
                float4 v = __ldg(c < C4 ? lat + c : rot + c);
                if (!live) v = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<uint2*>(dst + c * 4) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
            }
        }
    }

    float o[NO][4];
#pragma unroll
    for (int i = 0; i < NO; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
    const int g = lane >> 2, cq = lane & 3, mi = lane >> 3;
    const int row_a = rg * 16 + g, row_b = row_a + 8;
    const int hi0 = pos_first + row_a / HC, hi1 = pos_first + row_b / HC;      // the last key each of the two rows sees

    for (int kt = 0; kt < n_tiles; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                       // tile kt has landed (and the queries); tile kt - 1 is free
        if (kt + STAGES - 1 < n_tiles) load_tile((kt + STAGES - 1) % STAGES, key_begin + (kt + STAGES - 1) * KT, page_next);
        cp_async_commit();
        page_next = kt + STAGES < n_tiles ? page_of(key_begin + (kt + STAGES) * KT) : -1;
        const bf16* kt_s = k_s + (size_t)(kt % STAGES) * KT * LD;
        const int key0 = key_begin + kt * KT;
        // ---- s = q k^T for this warp's KW of the tile's 32 keys: NTW n-tiles of 8 keys, W / 16 k-steps; two sets of sums
        // (even and odd k-steps) keep the chains of dependent products short ----------------------------------------------------
        float s[NTW][4], s2[NTW][4];
#pragma unroll
        for (int i = 0; i < NTW; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = s2[i][0] = s2[i][1] = s2[i][2] = s2[i][3] = 0.f;
        {
            const bf16* qa = q_s + (size_t)(rg * 16 + (lane & 7) + (mi & 1) * 8) * LD + (mi >> 1) * 8;
            const int n_ks = W / 16;
            int ks = 0;
            if (NW == 2) {
                // one load brings 16 keys x 16 of the contraction
                const bf16* kb = kt_s + (size_t)(part * 16 + (mi >> 1) * 8 + (lane & 7)) * LD + (mi & 1) * 8;
#pragma unroll 2
                for (; ks + 2 <= n_ks; ks += 2) {
                    uint32_t a[4], b[4], a2[4], b2[4];
                    ldmatrix_x4(a, smem_addr(qa + ks * 16));
                    ldmatrix_x4(b, smem_addr(kb + ks * 16));
                    ldmatrix_x4(a2, smem_addr(qa + ks * 16 + 16));
                    ldmatrix_x4(b2, smem_addr(kb + ks * 16 + 16));
                    mma16816(s[0], a, b[0], b[1]);
                    mma16816(s[NTW - 1], a, b[2], b[3]);
                    mma16816(s2[0], a2, b2[0], b2[1]);
                    mma16816(s2[NTW - 1], a2, b2[2], b2[3]);
                }
                if (ks < n_ks) {
                    uint32_t a[4], b[4];
                    ldmatrix_x4(a, smem_addr(qa + ks * 16));
                    ldmatrix_x4(b, smem_addr(kb + ks * 16));
                    mma16816(s[0], a, b[0], b[1]);
                    mma16816(s[NTW - 1], a, b[2], b[3]);
                }
            } else {
                // one load brings 8 keys x 32 of the contraction: two k-steps
                const bf16* kb = kt_s + (size_t)(part * 8 + (lane & 7)) * LD + mi * 8;
#pragma unroll 2
                for (; ks + 2 <= n_ks; ks += 2) {
                    uint32_t a[4], a2[4], b[4];
                    ldmatrix_x4(a, smem_addr(qa + ks * 16));
                    ldmatrix_x4(a2, smem_addr(qa + ks * 16 + 16));
                    ldmatrix_x4(b, smem_addr(kb + ks * 16));
                    mma16816(s[0], a, b[0], b[1]);
                    mma16816(s2[0], a2, b[2], b[3]);
                }
                if (ks < n_ks) {
                    // the last, single k-step: the load's second half stays inside the row's padding and is not used
                    uint32_t a[4], b[4];
                    ldmatrix_x4(a, smem_addr(qa + ks * 16));
                    ldmatrix_x4(b, smem_addr(kt_s + (size_t)(part * 8 + (lane & 7)) * LD + (mi & 1) * 8 + ks * 16));
                    mma16816(s[0], a, b[0], b[1]);
                }
            }
#pragma unroll
            for (int i = 0; i < NTW; ++i)
#pragma unroll
                for (int x = 0; x < 4; ++x) s[i][x] += s2[i][x];
        }
        // ---- mask; the rows' maxima over all 32 keys, through the group's exchange -------------------------------------
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const int j = key0 + part * KW + nt * 8 + cq * 2 + x;
                const bool in = j >= k_lo && j < k_hi;
                const float a = (in && j <= hi0) ? s[nt][x] * scale_log2 : -CUDART_INF_F;
                const float b = (in && j <= hi1) ? s[nt][2 + x] * scale_log2 : -CUDART_INF_F;
                s[nt][x] = a, s[nt][2 + x] = b;
                mx0 = fmaxf(mx0, a), mx1 = fmaxf(mx1, b);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (cq == 0) xm[part * 16 + g] = mx0, xm[part * 16 + g + 8] = mx1;
        group_sync<NW>(rg);
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            mx0 = fmaxf(mx0, xm[w * 16 + g]);
            mx1 = fmaxf(mx1, xm[w * 16 + g + 8]);
        }
        const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
        const float sub0 = mn0 == -CUDART_INF_F ? 0.f : mn0, sub1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
        const float corr0 = exp2f(m[0] - sub0), corr1 = exp2f(m[1] - sub1);
        m[0] = mn0, m[1] = mn1;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pf[2][4];                                     // the tile's two k-steps of 16 keys
        {
            // this warp's weights go to their place among the fragments: n-tile t of the tile's four is registers
            // (t & 1) * 2, + 1 of k-step t >> 1
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) {
                const float p0 = exp2f(s[nt][0] - sub0), p1 = exp2f(s[nt][1] - sub0);
                const float p2 = exp2f(s[nt][2] - sub1), p3 = exp2f(s[nt][3] - sub1);
                sum0 += p0 + p1;
                sum1 += p2 + p3;
                const int t = part * NTW + nt;
                xp[((t >> 1) * 4 + (t & 1) * 2) * 32 + lane] = pack_bf16(p0, p1);
                xp[((t >> 1) * 4 + (t & 1) * 2 + 1) * 32 + lane] = pack_bf16(p2, p3);
            }
            group_sync<NW>(rg);
#pragma unroll
            for (int kk = 0; kk < 2; ++kk)
#pragma unroll
                for (int r = 0; r < 4; ++r) pf[kk][r] = xp[(kk * 4 + r) * 32 + lane];
        }
        l[0] = l[0] * corr0 + sum0;                            // partial sums (this thread's keys); added up at the end
        l[1] = l[1] * corr1 + sum1;
        // ---- o = o * corr + p v over this warp's half of the latent columns ------------------------------------------
        {
            const bf16* vb = kt_s + (size_t)((mi & 1) * 8 + (lane & 7)) * LD + part * CW + (mi >> 1) * 8;
#pragma unroll
            for (int np = 0; np < NO / 2; ++np) {
                float* o0 = o[np * 2];
                float* o1 = o[np * 2 + 1];
                o0[0] *= corr0; o0[1] *= corr0; o0[2] *= corr1; o0[3] *= corr1;
                o1[0] *= corr0; o1[1] *= corr0; o1[2] *= corr1; o1[3] *= corr1;
                uint32_t b[4];
                ldmatrix_x4_trans(b, smem_addr(vb + np * 16));
                mma16816(o0, pf[0], b[0], b[1]);
                mma16816(o1, pf[0], b[2], b[3]);
                ldmatrix_x4_trans(b, smem_addr(vb + (size_t)16 * LD + np * 16));
                mma16816(o0, pf[1], b[0], b[1]);
                mma16816(o1, pf[1], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    // ---- write out -----------------------------------------------------------------------------------------------------
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
    __syncthreads();                                           // (the exchange buffers of the last tile are free)
    if (cq == 0) xm[part * 16 + g] = l[0], xm[part * 16 + g + 8] = l[1];
    group_sync<NW>(rg);
    l[0] = l[1] = 0.f;                                         // every warp forms the same sum, in the same order
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        l[0] += xm[w * 16 + g];
        l[1] += xm[w * 16 + g + 8];
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int r = x ? row_b : row_a;
        const int tq = r / HC, n = head0 + r % HC;
        if (tq >= n_tq || n >= H) continue;
        const int t = tok0 + tq;
        if (splits == 1) {
            bf16* dst = out + ((size_t)n * head_rows + t) * C + part * CW;
            const float inv = 1.0f / l[x];
#pragma unroll
            for (int i = 0; i < NO; ++i)
                *reinterpret_cast<uint32_t*>(dst + i * 8 + cq * 2) = pack_bf16(o[i][2 * x] * inv, o[i][2 * x + 1] * inv);
        } else {
            const size_t item = ((size_t)t * H + n) * splits + split;
            float* dst = part_o + item * C + part * CW;
#pragma unroll
            for (int i = 0; i < NO; ++i)
                *reinterpret_cast<float2*>(dst + i * 8 + cq * 2) = make_float2(o[i][2 * x], o[i][2 * x + 1]);
            if (part == 0 && cq == 0) part_ml[item * 2] = m[x], part_ml[item * 2 + 1] = l[x];
        }
    }
}

// out[n, t, :] = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s, M = max_s m_s; one block per (token, head).  The
// ranges' weights are worked out once into shared memory; every range left a finite result (zeros where it saw no key),
// so the sums run over all of them without branches, several loads in flight, always in ascending order.
constexpr int MAX_SPLITS = 64;
__global__ void __launch_bounds__(256)
latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                    long long head_rows, int H, int C, int splits) {
    __shared__ float w_s[MAX_SPLITS];
    __shared__ float inv_s;
    const int t = blockIdx.x / H, n = blockIdx.x % H;
    const size_t item0 = ((size_t)t * H + n) * splits;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m0 = lane < splits ? part_ml[(item0 + lane) * 2] : -CUDART_INF_F;
        float m1 = lane + 32 < splits ? part_ml[(item0 + lane + 32) * 2] : -CUDART_INF_F;
        const float l0 = lane < splits ? part_ml[(item0 + lane) * 2 + 1] : 0.f;
        const float l1 = lane + 32 < splits ? part_ml[(item0 + lane + 32) * 2 + 1] : 0.f;
        const float M = warp_max(fmaxf(m0, m1));
        const float w0 = m0 == -CUDART_INF_F ? 0.f : exp2f(m0 - M), w1 = m1 == -CUDART_INF_F ? 0.f : exp2f(m1 - M);
        w_s[lane] = w0, w_s[lane + 32] = w1;
        // (the sum in a fixed order: lane by lane through the shuffle tree)
        const float L = warp_sum(w0 * l0 + w1 * l1);
        if (lane == 0) inv_s = 1.0f / L;
    }
    __syncthreads();
    const float inv = inv_s;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float* src = part_o + item0 * C + c;
        float acc = 0.f;
        int s = 0;
        for (; s + 8 <= splits; s += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = src[(size_t)(s + u) * C];
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = fmaf(w_s[s + u], v[u], acc);
        }
        for (; s < splits; ++s) acc = fmaf(w_s[s], src[(size_t)s * C], acc);
        out[((size_t)n * head_rows + t) * C + c] = __float2bfloat16_rn(acc * inv);
    }
}

template <int C, int ROWG, int STAGES, int NW>
int launch_one(const float* q_lat, const float* q_rot, long long head_rows, bf16* out, float* part_o, float* part_ml,
               const bf16* cache, const int* block_table, int max_blocks, const int* entry_q_start, const int* entry_q_len,
               const int* entry_pos0, int entry_first, int n_entries, int n_tiles, int TQ, int HC, int H, int R,
               int page_size, float scale, int chunk, int splits, cudaStream_t stream) {
    auto kern = latent_mma_kernel<C, ROWG, STAGES, NW>;
    const int LD = C + R + 8;
    const size_t sh = (size_t)(ROWG * 16 + STAGES * KT) * LD * sizeof(bf16) + (size_t)ROWG * (256 + 64) * 4;
    if (sh > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sh);
        if (err != cudaSuccess) {
            infero_set_error("latent attention: cannot get %zu bytes of shared memory: %s", sh, cudaGetErrorString(err));
            return 1;
        }
    }
    const dim3 grid(n_tiles, (H + HC - 1) / HC, splits);
    kern<<<grid, ROWG * NW * 32, sh, stream>>>(q_lat, q_rot, head_rows, out, part_o, part_ml, cache, block_table, max_blocks,
                                          entry_q_start, entry_q_len, entry_pos0, entry_first, n_entries, TQ, HC, H, R,
                                          page_size, scale * 1.4426950408889634f, chunk, splits);
    return 0;
}

}  // namespace

extern "C" {

// Sizes this kernel has instances for: a latent of 64, 128, 256 or 512, a rotated part that is a multiple of 16 and
// fits the shared memory beside it.
int infero_latent_mma_supported(int C, int R) {
    return (C == 64 || C == 128 || C == 256 || C == 512) && R >= 0 && R % 16 == 0 && R <= 128;
}

// Heads per CTA for H heads.
int infero_latent_mma_heads(int H) { return H <= 16 ? 16 : H <= 32 ? 32 : 64; }

// Entries [entry_first, n_entries) of the step; n_tiles = sum over them of ceil(q_len / TQ) (the host knows the lengths).
// single != 0: every entry brings one token (TQ = 1) and the keys are cut into `splits` ranges of `chunk` (a multiple of
// 32); with splits > 1 part_o float32 [tokens * H * splits * C] and part_ml [tokens * H * splits * 2] are scratch, indexed
// by the token's row in the step, and the merge runs behind.  Otherwise TQ = 64 / heads per CTA and splits = 1.
int infero_latent_attention_mma(const float* q_lat, const float* q_rot, long long head_rows, void* out, float* part_o,
                                float* part_ml, const void* cache, const int* block_table, int max_blocks,
                                const int* entry_q_start, const int* entry_q_len, const int* entry_pos0, int entry_first,
                                int n_entries, int n_tiles, int single, int H, int C, int R, int page_size, float scale,
                                int chunk, int splits, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    INFERO_REQUIRE(infero_latent_mma_supported(C, R), "latent attention: no tensor-core instance for a latent of %d + %d", C, R);
    INFERO_REQUIRE(splits <= MAX_SPLITS, "latent attention: %d ranges of keys, at most %d", splits, MAX_SPLITS);
    INFERO_REQUIRE(splits >= 1 && (splits == 1 || (single && chunk > 0 && chunk % KT == 0 && part_o && part_ml)),
                   "latent attention: %d splits of %d keys", splits, chunk);
    const int HC = infero_latent_mma_heads(H);
    const int TQ = single ? 1 : 64 / HC;
    const int rowg = single ? HC / 16 : 4;
    int rc = 1;
#define GO(C_, ROWG_, ST_)                                                                                              \
    rc = launch_one<C_, ROWG_, ST_, (C_ >= 256 && ROWG_ < 4 ? 4 : 2)>(q_lat, q_rot, head_rows, (bf16*)out, part_o, part_ml, (const bf16*)cache, block_table, \
                                    max_blocks, entry_q_start, entry_q_len, entry_pos0, entry_first, n_entries, n_tiles, TQ, \
                                    HC, H, R, page_size, scale, chunk, splits, stream)
#define BY_ROWS(C_)                                  \
    do {                                             \
        if (rowg == 1) GO(C_, 1, 2);                 \
        else if (rowg == 2) GO(C_, 2, 2);            \
        else GO(C_, 4, 2);                           \
    } while (0)
    if (C == 64) BY_ROWS(64);
    else if (C == 128) BY_ROWS(128);
    else if (C == 256) BY_ROWS(256);
    else BY_ROWS(512);
#undef BY_ROWS
#undef GO
    if (rc) return rc;
    if (splits > 1) {
        // the tokens of the leading single-token entries are the first rows of the step
        latent_merge_kernel<<<n_tiles * H, C >= 256 ? 256 : 128, 0, stream>>>(part_o, part_ml, (bf16*)out, head_rows, H, C, splits);
    }
    return infero_check_launch("latent_attention_mma");
}

}  // extern "C"

// The experts of many tokens as grouped matrix products on the warp-level tensor cores (bf16, 32-bit sums).
//
// align: the (token, choice) pairs are sorted by expert; every expert's run is padded to a whole number of
//   64-row tiles, so a tile belongs to one expert.  sorted_pair[r] is the pair (token * top + choice) in row
//   r, or -1 in padding; tile_expert[m] the expert of tile m, or -1 behind the last one.  The number of
//   tiles launched is a bound known on the host: ceil((pairs + experts * 63) / 64).
// up:   act[r, j] = silu(h_tok(r) . Wg_e[j]) * (h_tok(r) . Wu_e[j]) from the stacked [E, 2 ff, d] matrix whose
//       rows alternate gate_j, up_j: an accumulator's adjacent columns are such a pair.
// down: part[pair(r), i] = act[r] . Wd_e[i]     (float32 [tokens * top, d])
// combine: y[t] = sum_c w[t, c] * part[t * top + c] (+ gate[t] * shared[t]), choices in ascending order.
// A row's result does not depend on which rows share its tile.
//
// The product kernel: a CTA of four warps makes a 64 x 64 tile, K in steps of 32 through two shared-memory
// stages filled by cp.async; every warp owns 16 rows and all 64 columns (mma.sync m16n8k16).
#include "attn_common.cuh"

namespace {

using namespace attn;

constexpr int BM = 64, BN = 64, BK = 32, GT = 128;
constexpr int LDS = BK + 8;                 // padded row of a stage, in elements (80 bytes: 5 chunks, odd)
enum { EPI_SWIGLU = 0, EPI_SCATTER = 1 };

__global__ void moe_align_kernel(const int* __restrict__ top_idx, int n_pairs, int E, int top,
                                 int* __restrict__ sorted_pair, int* __restrict__ tile_expert, int max_tiles,
                                 int* __restrict__ a_rows /* token of each row, -1 in padding */) {
    extern __shared__ int sh[];
    int* count = sh;                        // [E]
    int* start = sh + E;                    // [E + 1], in rows, padded
    int* fill = start + E + 1;              // [E]
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0, fill[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&count[top_idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            at += (count[e] + BM - 1) / BM * BM;
        }
        start[E] = at;
    }
    __syncthreads();
    const int total = start[E];
    for (int r = threadIdx.x; r < max_tiles * BM; r += blockDim.x) sorted_pair[r] = -1, a_rows[r] = -1;
    for (int m = threadIdx.x; m < max_tiles; m += blockDim.x) {
        int e = -1;
        if (m * BM < total) {
            for (int k = 0; k < E; ++k)
                if (m * BM >= start[k] && m * BM < start[k + 1]) { e = k; break; }
        }
        tile_expert[m] = e;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = top_idx[p];
        const int r = start[e] + atomicAdd(&fill[e], 1);
        sorted_pair[r] = p;
        a_rows[r] = p / top;
    }
}

template <int EPI>
__global__ void __launch_bounds__(GT)
grouped_gemm_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ a_rows, const bf16* __restrict__ B,
                    const int* __restrict__ tile_expert, int N, int K, void* __restrict__ out, int ldo,
                    const int* __restrict__ out_rows) {
    __shared__ __align__(16) bf16 As[2][BM * LDS];
    __shared__ __align__(16) bf16 Bs[2][BN * LDS];
    const int mt = blockIdx.x, nt = blockIdx.y;
    const int e = tile_expert[mt];
    if (e < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bf16* Be = B + (size_t)e * N * K;

    auto load = [&](int stage, int k0) {
        for (int i = tid; i < BM * (BK / 8); i += GT) {
            const int r = i / (BK / 8), c = i % (BK / 8);
            const int k = k0 + c * 8;
            bf16* dst = &As[stage][r * LDS + c * 8];
            const int ar = a_rows ? a_rows[mt * BM + r] : mt * BM + r;
            if (ar >= 0 && k < K) cp_async16(smem_addr(dst), A + (size_t)ar * lda + k);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        for (int i = tid; i < BN * (BK / 8); i += GT) {
            const int r = i / (BK / 8), c = i % (BK / 8);
            const int k = k0 + c * 8, n = nt * BN + r;
            bf16* dst = &Bs[stage][r * LDS + c * 8];
            if (n < N && k < K) cp_async16(smem_addr(dst), Be + (size_t)n * K + k);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };

    float acc[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int n_k = (K + BK - 1) / BK;
    load(0, 0);
    for (int kt = 0; kt < n_k; ++kt) {
        if (kt + 1 < n_k) load((kt + 1) & 1, (kt + 1) * BK);
        else cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* as = As[kt & 1];
        const bf16* bs = Bs[kt & 1];
        const int mi = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, smem_addr(as + (warp * 16 + (lane & 7) + (mi & 1) * 8) * LDS + ks * 16 + (mi >> 1) * 8));
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, smem_addr(bs + (np * 16 + (mi >> 1) * 8 + (lane & 7)) * LDS + ks * 16 + (mi & 1) * 8));
                mma16816(acc[np * 2], a, b[0], b[1]);
                mma16816(acc[np * 2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    const int g = lane >> 2, c = lane & 3;
    const int r0 = mt * BM + warp * 16 + g, r1 = r0 + 8;
    if (EPI == EPI_SWIGLU) {
        bf16* o = (bf16*)out;
#pragma unroll
        for (int n8 = 0; n8 < BN / 8; ++n8) {
            const int col = nt * BN + n8 * 8 + c * 2;            // even: gate, col + 1: up
            if (col + 1 < N) {
                const float g0 = acc[n8][0], u0 = acc[n8][1], g1 = acc[n8][2], u1 = acc[n8][3];
                o[(size_t)r0 * ldo + col / 2] = __float2bfloat16_rn(g0 / (1.0f + expf(-g0)) * u0);
                o[(size_t)r1 * ldo + col / 2] = __float2bfloat16_rn(g1 / (1.0f + expf(-g1)) * u1);
            }
        }
    } else {
        float* o = (float*)out;
        const int p0 = out_rows[r0], p1 = out_rows[r1];
#pragma unroll
        for (int n8 = 0; n8 < BN / 8; ++n8) {
            const int col = nt * BN + n8 * 8 + c * 2;
            if (col < N) {
                if (p0 >= 0) o[(size_t)p0 * ldo + col] = acc[n8][0];
                if (p1 >= 0) o[(size_t)p1 * ldo + col] = acc[n8][2];
            }
            if (col + 1 < N) {
                if (p0 >= 0) o[(size_t)p0 * ldo + col + 1] = acc[n8][1];
                if (p1 >= 0) o[(size_t)p1 * ldo + col + 1] = acc[n8][3];
            }
        }
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ part, const float* __restrict__ top_w,
                                   const float* __restrict__ shared, const float* __restrict__ shared_gate,
                                   float* __restrict__ y, int d, int top) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < top; ++c) acc = fmaf(top_w[t * top + c], part[(t * top + c) * d + i], acc);
        if (shared) acc = fmaf(shared_gate ? shared_gate[t] : 1.0f, shared[t * d + i], acc);
        y[t * d + i] = acc;
    }
}

}  // namespace

extern "C" {

int infero_moe_grouped_tiles(int n_pairs, int E) { return (n_pairs + E * (BM - 1) + BM - 1) / BM; }

// Scratch (the caller allocates): sorted_pair, a_rows int32 [tiles * 64]; tile_expert int32 [tiles];
// act bf16 [tiles * 64, ff]; part float32 [tokens * top, d].
int infero_moe_experts_grouped(const void* h, int h_stride, const void* gate_up, const void* down, const int* top_idx,
                               const float* top_w, const float* shared, const float* shared_gate, int* sorted_pair,
                               int* a_rows, int* tile_expert, void* act, float* part, float* y, int n_tokens, int d,
                               int ff, int E, int top, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(d % 8 == 0 && ff % 8 == 0 && h_stride % 8 == 0, "moe grouped: widths %d / %d must be multiples of 8", d, ff);
    const int n_pairs = n_tokens * top, tiles = infero_moe_grouped_tiles(n_pairs, E);
    const size_t sh = (size_t)(3 * E + 1) * sizeof(int);
    INFERO_REQUIRE(sh <= 48 * 1024, "moe grouped: %d experts are too many", E);
    moe_align_kernel<<<1, 1024, sh, stream>>>(top_idx, n_pairs, E, top, sorted_pair, tile_expert, tiles, a_rows);
    grouped_gemm_kernel<EPI_SWIGLU><<<dim3(tiles, (2 * ff + BN - 1) / BN), GT, 0, stream>>>(
        (const bf16*)h, h_stride, a_rows, (const bf16*)gate_up, tile_expert, 2 * ff, d, act, ff, nullptr);
    grouped_gemm_kernel<EPI_SCATTER><<<dim3(tiles, (d + BN - 1) / BN), GT, 0, stream>>>(
        (const bf16*)act, ff, nullptr, (const bf16*)down, tile_expert, d, ff, part, d, sorted_pair);
    moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(part, top_w, shared, shared_gate, y, d, top);
    return infero_check_launch("moe_experts_grouped");
}

}  // extern "C"

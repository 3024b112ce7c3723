// The experts of many tokens as grouped matrix products on the warp-level tensor cores (bf16, 32-bit sums).
//
// align: the (token, choice) pairs are sorted by expert; every expert's run is padded to a whole number of
//   tiles of 64 or 128 rows, so a tile belongs to one expert.  sorted_pair[r] is the pair (token * top + choice) in row
//   r, or -1 in padding; tile_expert[m] the expert of tile m, or -1 behind the last one.  The number of
//   tiles launched is a bound known on the host: ceil((pairs + experts * (rows - 1)) / rows).
// up:   act[r, j] = glu(h_tok(r) . Wg_e[j], h_tok(r) . Wu_e[j]) (a gated activation of common.cuh) from the stacked [E, 2 ff, d] matrix whose
//       rows alternate gate_j, up_j: an accumulator's adjacent columns are such a pair.
// down: part[pair(r), i] = act[r] . Wd_e[i]     (float32 [tokens * top, d])
// combine: y[t] = sum_c w[t, c] * part[t * top + c] (+ gate[t] * shared[t]), choices in ascending order.
// A row's result does not depend on which rows share its tile.
//
// The product kernel (mma.sync m16n8k16, K in steps of 32 through shared-memory stages filled by cp.async): when an
// expert gets about a tile's worth of pairs, a CTA of eight warps makes a 128 x 128 tile through three stages (a warp
// owns 32 x 64); else four warps make a 64 x 64 tile through two stages (a warp owns 16 x 64).
#include "attn_common.cuh"

namespace {

using namespace attn;

constexpr int BK = 32;
constexpr int LDS = BK + 8;                 // padded row of a stage, in elements (80 bytes: 5 chunks, odd)
enum { EPI_SWIGLU = 0, EPI_SCATTER = 1 };

__global__ void moe_align_kernel(const int* __restrict__ top_idx, int n_pairs, int E, int top,
                                 int* __restrict__ sorted_pair, int* __restrict__ tile_expert, int max_tiles,
                                 int* __restrict__ a_rows /* token of each row, -1 in padding */, int BM,
                                 int* __restrict__ pair_row /* row of each pair, or null */) {
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
    if (threadIdx.x == 0) tile_expert[max_tiles] = total;       // rows in use (tile_expert has max_tiles + 1 entries)
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = top_idx[p];
        const int r = start[e] + atomicAdd(&fill[e], 1);
        sorted_pair[r] = p;
        a_rows[r] = p / top;
        if (pair_row) pair_row[p] = r;
    }
}

// xs[r, :] = h[a_rows[r], :] (zeros where a_rows[r] < 0); rows of d bf16, d a multiple of 8.  With pair_w the row is
// multiplied by the weight of the pair it stands for (pair_w[sorted_pair[r]]) and rounded once.
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ h, int h_stride, const int* __restrict__ a_rows,
                                       bf16* __restrict__ xs, int d, const int* __restrict__ sorted_pair,
                                       const float* __restrict__ pair_w) {
    const size_t r = blockIdx.x;
    const int src = a_rows[r];
    const float f = (pair_w && src >= 0) ? pair_w[sorted_pair[r]] : 1.0f;
    for (int c = threadIdx.x; c < d / 8; c += blockDim.x) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (src >= 0) v = *reinterpret_cast<const uint4*>(h + (size_t)src * h_stride + c * 8);
        if (pair_w) {
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
                const __nv_bfloat162 p2 = __floats2bfloat162_rn(lo * f, hi * f);
                w[j] = *reinterpret_cast<const uint32_t*>(&p2);
            }
            v = make_uint4(w[0], w[1], w[2], w[3]);
        }
        *reinterpret_cast<uint4*>(xs + r * d + c * 8) = v;
    }
}

// y[t] = sum_c w[t, c] * rows[pair_row[t * top + c]] (+ gate[t] * shared[t]), choices in ascending order
__global__ void moe_combine_rows_kernel(const float* __restrict__ rows, const int* __restrict__ pair_row,
                                        const float* __restrict__ top_w, const float* __restrict__ shared,
                                        const float* __restrict__ shared_gate, float* __restrict__ y, int d, int top) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < top; ++c) {
            const float v = rows[(size_t)pair_row[t * top + c] * d + i];
            acc = top_w ? fmaf(top_w[t * top + c], v, acc) : acc + v;
        }
        if (shared) acc = fmaf(shared_gate ? shared_gate[t] : 1.0f, shared[t * d + i], acc);
        y[t * d + i] = acc;
    }
}

// TM x TN tile by WM x WN warps (a warp makes (TM / WM) x (TN / WN)), K in steps of 32 through STAGES stages.
template <int EPI, int TM, int TN, int WM, int WN, int STAGES>
__global__ void __launch_bounds__(WM * WN * 32)
grouped_gemm_kernel(const bf16* __restrict__ A, int lda, const int* __restrict__ a_rows, const bf16* __restrict__ B,
                    const int* __restrict__ tile_expert, int N, int K, void* __restrict__ out, int ldo,
                    const int* __restrict__ out_rows, int act_kind, float act_limit, float act_alpha) {
    constexpr int NT = WM * WN * 32, MI = TM / WM / 16, NI = TN / WN / 8;
    extern __shared__ __align__(16) uint8_t gsm[];
    bf16* As = reinterpret_cast<bf16*>(gsm);                    // [STAGES][TM * LDS]
    bf16* Bs = As + STAGES * TM * LDS;                          // [STAGES][TN * LDS]
    const int mt = blockIdx.x, nt = blockIdx.y;
    const int e = tile_expert[mt];
    if (e < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp % WM, wn = warp / WM;
    const bf16* Be = B + (size_t)e * N * K;

    auto load = [&](int stage, int k0) {
        for (int i = tid; i < TM * (BK / 8); i += NT) {
            const int r = i / (BK / 8), c = i % (BK / 8);
            const int k = k0 + c * 8;
            bf16* dst = As + stage * TM * LDS + r * LDS + c * 8;
            const int ar = a_rows ? a_rows[mt * TM + r] : mt * TM + r;
            if (ar >= 0 && k < K) cp_async16(smem_addr(dst), A + (size_t)ar * lda + k);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        for (int i = tid; i < TN * (BK / 8); i += NT) {
            const int r = i / (BK / 8), c = i % (BK / 8);
            const int k = k0 + c * 8, n = nt * TN + r;
            bf16* dst = Bs + stage * TN * LDS + r * LDS + c * 8;
            if (n < N && k < K) cp_async16(smem_addr(dst), Be + (size_t)n * K + k);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    };

    float acc[MI][NI][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    const int n_k = (K + BK - 1) / BK;
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < n_k) load(st, st * BK);
        cp_async_commit();
    }
    for (int kt = 0; kt < n_k; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                        // stage kt has landed; stage kt-1 is free for all
        if (kt + STAGES - 1 < n_k) load((kt + STAGES - 1) % STAGES, (kt + STAGES - 1) * BK);
        cp_async_commit();
        const bf16* as = As + (kt % STAGES) * TM * LDS;
        const bf16* bs = Bs + (kt % STAGES) * TN * LDS;
        const int mi = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            uint32_t a[MI][4];
#pragma unroll
            for (int i = 0; i < MI; ++i)
                ldmatrix_x4(a[i], smem_addr(as + ((wm * MI + i) * 16 + (lane & 7) + (mi & 1) * 8) * LDS + ks * 16 + (mi >> 1) * 8));
#pragma unroll
            for (int np = 0; np < NI / 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, smem_addr(bs + (wn * NI * 8 + np * 16 + (mi >> 1) * 8 + (lane & 7)) * LDS + ks * 16 + (mi & 1) * 8));
#pragma unroll
                for (int i = 0; i < MI; ++i) {
                    mma16816(acc[i][np * 2], a[i], b[0], b[1]);
                    mma16816(acc[i][np * 2 + 1], a[i], b[2], b[3]);
                }
            }
        }
    }
    const int g = lane >> 2, c = lane & 3;
#pragma unroll
    for (int i = 0; i < MI; ++i) {
        const int r0 = mt * TM + (wm * MI + i) * 16 + g, r1 = r0 + 8;
        if (EPI == EPI_SWIGLU) {
            bf16* o = (bf16*)out;
#pragma unroll
            for (int n8 = 0; n8 < NI; ++n8) {
                const int col = nt * TN + wn * NI * 8 + n8 * 8 + c * 2;      // even: gate, col + 1: up
                if (col + 1 < N) {
                    const float g0 = acc[i][n8][0], u0 = acc[i][n8][1], g1 = acc[i][n8][2], u1 = acc[i][n8][3];
                    o[(size_t)r0 * ldo + col / 2] = __float2bfloat16_rn(glu_act(g0, u0, act_kind, act_limit, act_alpha));
                    o[(size_t)r1 * ldo + col / 2] = __float2bfloat16_rn(glu_act(g1, u1, act_kind, act_limit, act_alpha));
                }
            }
        } else {
            float* o = (float*)out;
            const int p0 = out_rows[r0], p1 = out_rows[r1];
#pragma unroll
            for (int n8 = 0; n8 < NI; ++n8) {
                const int col = nt * TN + wn * NI * 8 + n8 * 8 + c * 2;
                if (col < N) {
                    if (p0 >= 0) o[(size_t)p0 * ldo + col] = acc[i][n8][0];
                    if (p1 >= 0) o[(size_t)p1 * ldo + col] = acc[i][n8][2];
                }
                if (col + 1 < N) {
                    if (p0 >= 0) o[(size_t)p0 * ldo + col + 1] = acc[i][n8][1];
                    if (p1 >= 0) o[(size_t)p1 * ldo + col + 1] = acc[i][n8][3];
                }
            }
        }
    }
}

template <int EPI, int TM, int TN, int WM, int WN, int STAGES>
void launch_grouped(const bf16* A, int lda, const int* a_rows, const bf16* B, const int* tile_expert, int tiles, int N, int K,
                    void* out, int ldo, const int* out_rows, cudaStream_t stream, int act_kind = GLU_SILU, float act_limit = 0.f,
                    float act_alpha = 1.f) {
    auto kern = grouped_gemm_kernel<EPI, TM, TN, WM, WN, STAGES>;
    const int smem = STAGES * (TM + TN) * LDS * 2;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    kern<<<dim3(tiles, (N + TN - 1) / TN), WM * WN * 32, smem, stream>>>(A, lda, a_rows, B, tile_expert, N, K, out, ldo, out_rows,
                                                                         act_kind, act_limit, act_alpha);
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

// Rows of a tile: 128 when an expert gets about a tile's worth of pairs, else 64.
int infero_moe_grouped_tile_rows(int n_pairs, int E) { return n_pairs >= 96 * E ? 128 : 64; }
int infero_moe_grouped_tiles(int n_pairs, int E) {
    const int BM = infero_moe_grouped_tile_rows(n_pairs, E);
    return (n_pairs + E * (BM - 1) + BM - 1) / BM;
}

// Scratch (the caller allocates), with R = tiles * tile rows: sorted_pair, a_rows int32 [R]; tile_expert int32 [tiles + 1];
// act bf16 [R, ff]; part float32 [tokens * top, d].
int infero_moe_experts_grouped(const void* h, int h_stride, const void* gate_up, const void* down, const int* top_idx,
                               const float* top_w, const float* shared, const float* shared_gate, int* sorted_pair,
                               int* a_rows, int* tile_expert, void* act, float* part, float* y, int n_tokens, int d,
                               int ff, int E, int top, int act_kind, float act_limit, float act_alpha, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(d % 8 == 0 && ff % 8 == 0 && h_stride % 8 == 0, "moe grouped: widths %d / %d must be multiples of 8", d, ff);
    const int n_pairs = n_tokens * top, tiles = infero_moe_grouped_tiles(n_pairs, E);
    const int BM = infero_moe_grouped_tile_rows(n_pairs, E);
    const size_t sh = (size_t)(3 * E + 1) * sizeof(int);
    INFERO_REQUIRE(sh <= 48 * 1024, "moe grouped: %d experts are too many", E);
    moe_align_kernel<<<1, 1024, sh, stream>>>(top_idx, n_pairs, E, top, sorted_pair, tile_expert, tiles, a_rows, BM, nullptr);
    if (BM == 128) {
        launch_grouped<EPI_SWIGLU, 128, 128, 4, 2, 3>((const bf16*)h, h_stride, a_rows, (const bf16*)gate_up, tile_expert, tiles,
                                                      2 * ff, d, act, ff, nullptr, stream, act_kind, act_limit, act_alpha);
        launch_grouped<EPI_SCATTER, 128, 128, 4, 2, 3>((const bf16*)act, ff, nullptr, (const bf16*)down, tile_expert, tiles,
                                                       d, ff, part, d, sorted_pair, stream);
    } else {
        launch_grouped<EPI_SWIGLU, 64, 64, 4, 1, 2>((const bf16*)h, h_stride, a_rows, (const bf16*)gate_up, tile_expert, tiles,
                                                    2 * ff, d, act, ff, nullptr, stream, act_kind, act_limit, act_alpha);
        launch_grouped<EPI_SCATTER, 64, 64, 4, 1, 2>((const bf16*)act, ff, nullptr, (const bf16*)down, tile_expert, tiles,
                                                     d, ff, part, d, sorted_pair, stream);
    }
    moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(part, top_w, shared, shared_gate, y, d, top);
    return infero_check_launch("moe_experts_grouped");
}

// ---- the pieces around grouped products on the tcgen05 kernel (128-row tiles) ----------------------------------
int infero_moe_tc_tiles(int n_pairs, int E) { return (n_pairs + E * 127 + 127) / 128; }

// sorted_pair, a_rows int32 [tiles * 128]; tile_expert int32 [tiles + 1]; pair_row int32 [tokens * top];
// xs bf16 [tiles * 128, d]: the tokens' rows in sorted order.
// pair_w (float32 [tokens * top] or null): a row of xs is its token's row times the weight of its pair.
int infero_moe_tc_prepare_scaled(const void* h, int h_stride, const int* top_idx, int* sorted_pair, int* a_rows,
                                 int* tile_expert, int* pair_row, void* xs, int n_tokens, int d, int E, int top,
                                 const float* pair_w, cudaStream_t stream) {
    INFERO_REQUIRE(d % 8 == 0 && h_stride % 8 == 0, "moe: width %d must be a multiple of 8", d);
    const int n_pairs = n_tokens * top, tiles = infero_moe_tc_tiles(n_pairs, E);
    const size_t sh = (size_t)(3 * E + 1) * sizeof(int);
    INFERO_REQUIRE(sh <= 48 * 1024, "moe grouped: %d experts are too many", E);
    moe_align_kernel<<<1, 1024, sh, stream>>>(top_idx, n_pairs, E, top, sorted_pair, tile_expert, tiles, a_rows, 128, pair_row);
    moe_gather_rows_kernel<<<tiles * 128, 128, 0, stream>>>((const bf16*)h, h_stride, a_rows, (bf16*)xs, d, sorted_pair, pair_w);
    return infero_check_launch("moe_tc_prepare");
}

int infero_moe_tc_prepare(const void* h, int h_stride, const int* top_idx, int* sorted_pair, int* a_rows, int* tile_expert,
                          int* pair_row, void* xs, int n_tokens, int d, int E, int top, cudaStream_t stream) {
    return infero_moe_tc_prepare_scaled(h, h_stride, top_idx, sorted_pair, a_rows, tile_expert, pair_row, xs, n_tokens, d, E,
                                        top, nullptr, stream);
}

int infero_moe_tc_combine(const float* rows, const int* pair_row, const float* top_w, const float* shared,
                          const float* shared_gate, float* y, int n_tokens, int d, int top, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    moe_combine_rows_kernel<<<n_tokens, 256, 0, stream>>>(rows, pair_row, top_w, shared, shared_gate, y, d, top);
    return infero_check_launch("moe_tc_combine");
}

}  // extern "C"

// Attention whose keys and values are made from one small cached vector per token ("latent attention").
//
// Per token the layer's input product gives a query of H heads, each [D plain | R rotated] wide, and one row of
// C + R numbers: the first C, RMS-normed with a weight, are the latent c; the last R are a rotated key part shared by
// all heads.  Head n's key is [Wuk_n c | rotated part], its value Wuv_n c.  Only the row [c | rotated part] is cached
// (one "kv head" of width C + R; the value of a key is the first C columns of the same row), and the two
// up-projections move to the query side:
//     q_n . k_n = (Wuk_n^T q_n,plain) . c + q_n,rot . k_rot        out_n = Wuv_n (sum_j p_j c_j)
// so a step runs  prepare -> per-head product with Wuk^T -> attention over the latent rows -> per-head product with
// Wuv -> finish (optional sigmoid gate per head, heads side by side).  The per-head products are the engine's
// matrix-product kernels; queries and results are kept head-major, [H, rows, width], for them.
//
// prepare: per token one block for the latent row and one per group of heads.  c = row[:C] / sqrt(mean(row[:C]^2) + eps) * w (32-bit); the first `rot` of the R
//   rotated coordinates of the key part and of every head's query turn by position * freq[i], cos and sin times
//   `amp` (a 64-bit frequency table and the amplitude come from the host, so any scaling of the frequencies is the host's);
//   pairing 0: coordinate i with i + rot/2, pairing 1: 2i with 2i + 1.  The row [c | key part] goes to the token's
//   page, the plain query parts to q_plain (the element type of the step) and the rotated ones to q_rot (float32).
// attention (this file: the any-type kernel, one warp per (token, head); keys in ascending chunks of 32 aligned to
//   absolute positions, running maximum and sum in 32-bit, so a token's arithmetic depends on its own position only).
// finish: out[t, n * V + v] = val[n, t, v] * sigmoid(gate[t, n]).
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int PREP_THREADS = 128;

// The angle is position times frequency in 64-bit, brought into [-pi, pi] there and only then rounded: a 32-bit product
// is off by its own size times 2^-24, which at position 1,000 is already 6e-5 of a turn's worth of radians.
__device__ __forceinline__ void turn(float a, float b, double ang, float amp, float& ra, float& rb) {
    const double two_pi = 6.283185307179586476925286766559;
    ang -= two_pi * rint(ang / two_pi);
    float s, c;
    sincosf((float)ang, &s, &c);
    s *= amp, c *= amp;
    ra = a * c - b * s;
    rb = b * c + a * s;
}

// element i of a rotated part of width R: what it becomes at position p
__device__ __forceinline__ float rotated(const float* __restrict__ part, int i, int rot, int pairing, int pos,
                                         const double* __restrict__ freq, float amp) {
    if (i >= rot) return part[i];
    int ia, ib;
    if (pairing) ia = i & ~1, ib = ia + 1;
    else ia = i < rot / 2 ? i : i - rot / 2, ib = ia + rot / 2;
    const int pair = pairing ? i >> 1 : ia;
    float ra, rb;
    turn(part[ia], part[ib], (double)pos * freq[pair], amp, ra, rb);
    return i == ia ? ra : rb;
}

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
latent_prepare_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ q_src, int q_stride,
                      int q_off, int kv_off,
                      const float* __restrict__ norm_w, float eps, const double* __restrict__ freq, int rot, int pairing,
                      float amp, const int* __restrict__ positions, const int* __restrict__ tok_entry,
                      const int* __restrict__ block_table, int max_blocks, int page_size, T* __restrict__ cache,
                      int write_cache, T* __restrict__ q_plain, float* __restrict__ q_rot, long long head_rows,
                      int H, int D, int R, int C, int heads_per_block) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * proj_stride;
    const int pos = positions[t];
    if (blockIdx.y == 0) {
        // the latent row
        if (!write_cache) return;
        const float* kv = row + kv_off;
        float sq = 0.f;
        for (int i = threadIdx.x; i < C; i += blockDim.x) sq = fmaf(kv[i], kv[i], sq);
        const float rstd = 1.0f / sqrtf(block_sum(sq, red) / (float)C + eps);
        const int p = positions[t];
        const int page = block_table[(size_t)tok_entry[t] * max_blocks + p / page_size];
        T* dst = cache + ((size_t)page * page_size + (p % page_size)) * (C + R);
        for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = from_f32<T>(kv[i] * rstd * norm_w[i]);
        for (int i = threadIdx.x; i < R; i += blockDim.x) dst[C + i] = from_f32<T>(rotated(kv + C, i, rot, pairing, pos, freq, amp));
        return;
    }
    // the queries of heads [n0, n1)
    const int n0 = (blockIdx.y - 1) * heads_per_block, n1 = min(H, n0 + heads_per_block);
    const float* q = q_src + (size_t)t * q_stride + q_off;
    for (int i = n0 * D + threadIdx.x; i < n1 * D; i += blockDim.x) {
        const int n = i / D, c = i % D;
        q_plain[((size_t)n * head_rows + t) * D + c] = from_f32<T>(q[(size_t)n * (D + R) + c]);
    }
    for (int i = n0 * R + threadIdx.x; i < n1 * R; i += blockDim.x) {
        const int n = i / R, c = i % R;
        q_rot[((size_t)n * head_rows + t) * R + c] = rotated(q + (size_t)n * (D + R) + D, c, rot, pairing, pos, freq, amp);
    }
}

constexpr int WARPS = 4;
constexpr int MAX_C = 1024;           // widest latent the any-type kernel keeps in registers (32 per lane)

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_generic_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, long long head_rows,
                                T* __restrict__ out, const T* __restrict__ cache, const int* __restrict__ block_table,
                                int max_blocks, const int* __restrict__ tok_entry, const int* __restrict__ positions,
                                int tok_first, int n_tokens, int H, int C, int R, int page_size, float scale) {
    extern __shared__ float q_s[];                       // [WARPS][C + R]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = tok_first + (int)(item / H), n = (int)(item % H);
    const int W = C + R;
    float* qs = q_s + (size_t)warp * W;
    const size_t qrow = (size_t)n * head_rows + t;
    for (int i = lane; i < C; i += 32) qs[i] = q_lat[qrow * C + i];
    for (int i = lane; i < R; i += 32) qs[C + i] = q_rot[qrow * R + i];
    __syncwarp();
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_entry[t] * max_blocks;

    float m = -CUDART_INF_F, l = 0.f;
    float acc[MAX_C / 32];
#pragma unroll
    for (int i = 0; i < MAX_C / 32; ++i) acc[i] = 0.f;
    for (int j0 = 0; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        long long row = -1;
        float s = -CUDART_INF_F;
        if (j <= pos) {
            const int page = table[j / page_size];
            if (page >= 0) {
                row = ((long long)page * page_size + (j % page_size)) * W;
                const T* kr = cache + row;
                float d = 0.f;
                for (int i = 0; i < W; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
                s = d * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -CUDART_INF_F) continue;
        const float p = (row >= 0) ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_C / 32; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            if (rj < 0) continue;
            const T* vr = cache + rj;
#pragma unroll
            for (int i = 0; i < MAX_C / 32; ++i) {
                const int dd = i * 32 + lane;
                if (dd < C) acc[i] = fmaf(pj, to_f32(vr[dd]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + qrow * C;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_C / 32; ++i) {
        const int dd = i * 32 + lane;
        if (dd < C) orow[dd] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
__global__ void latent_finish_kernel(const float* __restrict__ val, long long head_rows, const float* __restrict__ gate,
                                     int gate_stride, T* __restrict__ out, int out_stride, int H, int V) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H * V; i += blockDim.x) {
        const int n = i / V, v = i % V;
        float x = val[((size_t)n * head_rows + t) * V + v];
        if (gate) x *= 1.0f / (1.0f + expf(-gate[t * gate_stride + n]));
        out[t * out_stride + i] = from_f32<T>(x);
    }
}

}  // namespace

extern "C" {

// proj float32 [T, proj_stride]: the C + R columns of the latent row from kv_off.  q_src float32 [T, q_stride]: the
// query's H * (D + R) columns from q_off (the same array as proj where one product gives both, another where the queries
// come from a product of their own).  cache [pages, 1, page, C + R]; q_plain [H, head_rows, D] of the cache's type; q_rot
// float32 [H, head_rows, R] (R may be 0: no rotated part).
int infero_latent_prepare_from(const float* proj, int proj_stride, const float* q_src, int q_stride, int q_off, int kv_off,
                               const float* norm_w, float eps,
                          const double* freq, int rot, int pairing, float amp, const int* positions, const int* tok_entry,
                          const int* block_table, int max_blocks, int page_size, void* cache, int dtype, int write_cache,
                          void* q_plain, float* q_rot, long long head_rows, int n_tokens, int H, int D, int R, int C,
                          cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(rot >= 0 && rot <= R && rot % 2 == 0, "latent attention: %d rotated coordinates of %d", rot, R);
    INFERO_REQUIRE(head_rows >= n_tokens, "latent attention: %lld rows per head for %d tokens", head_rows, n_tokens);
    // one block for a token's latent row, and one per group of heads (all heads in one block where tokens alone fill
    // the multiprocessors)
    const int heads_per_block = n_tokens >= 512 ? H : max(1, H / 8);
    const dim3 grid(n_tokens, 1 + (H + heads_per_block - 1) / heads_per_block);
    if (dtype == INFERO_F32)
        latent_prepare_kernel<float><<<grid, PREP_THREADS, 0, stream>>>(proj, proj_stride, q_src, q_stride, q_off, kv_off, norm_w, eps, freq,
            rot, pairing, amp, positions, tok_entry, block_table, max_blocks, page_size, (float*)cache, write_cache,
            (float*)q_plain, q_rot, head_rows, H, D, R, C, heads_per_block);
    else
        latent_prepare_kernel<bf16><<<grid, PREP_THREADS, 0, stream>>>(proj, proj_stride, q_src, q_stride, q_off, kv_off, norm_w, eps, freq,
            rot, pairing, amp, positions, tok_entry, block_table, max_blocks, page_size, (bf16*)cache, write_cache,
            (bf16*)q_plain, q_rot, head_rows, H, D, R, C, heads_per_block);
    return infero_check_launch("latent_prepare");
}

int infero_latent_prepare(const float* proj, int proj_stride, int q_off, int kv_off, const float* norm_w, float eps,
                          const double* freq, int rot, int pairing, float amp, const int* positions, const int* tok_entry,
                          const int* block_table, int max_blocks, int page_size, void* cache, int dtype, int write_cache,
                          void* q_plain, float* q_rot, long long head_rows, int n_tokens, int H, int D, int R, int C,
                          cudaStream_t stream) {
    return infero_latent_prepare_from(proj, proj_stride, proj, proj_stride, q_off, kv_off, norm_w, eps, freq, rot, pairing, amp,
                                      positions, tok_entry, block_table, max_blocks, page_size, cache, dtype, write_cache,
                                      q_plain, q_rot, head_rows, n_tokens, H, D, R, C, stream);
}

// q_lat float32 [H, head_rows, C] (the plain query parts carried through Wuk^T), q_rot float32 [H, head_rows, R];
// out [H, head_rows, C] of the cache's type: softmax-weighted sums of the latent rows.  Tokens tok_first .. + n_tokens.
int infero_latent_attention_generic(const float* q_lat, const float* q_rot, long long head_rows, void* out, const void* cache,
                                    int dtype, const int* block_table, int max_blocks, const int* tok_entry,
                                    const int* positions, int tok_first, int n_tokens, int H, int C, int R, int page_size,
                                    float scale, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(C >= 1 && C <= MAX_C, "latent attention: latent width %d outside 1..%d", C, MAX_C);
    const size_t sh = (size_t)WARPS * (C + R) * sizeof(float);
    INFERO_REQUIRE(sh <= 48 * 1024, "latent attention: key width %d too large", C + R);
    const long long items = (long long)n_tokens * H;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (dtype == INFERO_F32)
        latent_attention_generic_kernel<float><<<blocks, WARPS * 32, sh, stream>>>(q_lat, q_rot, head_rows, (float*)out,
            (const float*)cache, block_table, max_blocks, tok_entry, positions, tok_first, n_tokens, H, C, R, page_size, scale);
    else
        latent_attention_generic_kernel<bf16><<<blocks, WARPS * 32, sh, stream>>>(q_lat, q_rot, head_rows, (bf16*)out,
            (const bf16*)cache, block_table, max_blocks, tok_entry, positions, tok_first, n_tokens, H, C, R, page_size, scale);
    return infero_check_launch("latent_attention_generic");
}

// val float32 [H, head_rows, V]; gate float32 (row stride gate_stride, one column per head) or null; out [T, H * V].
int infero_latent_finish(const float* val, long long head_rows, const float* gate, int gate_stride, void* out,
                         int out_stride, int dtype, int n_tokens, int H, int V, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    if (dtype == INFERO_F32)
        latent_finish_kernel<float><<<n_tokens, 256, 0, stream>>>(val, head_rows, gate, gate_stride, (float*)out, out_stride, H, V);
    else
        latent_finish_kernel<bf16><<<n_tokens, 256, 0, stream>>>(val, head_rows, gate, gate_stride, (bf16*)out, out_stride, H, V);
    return infero_check_launch("latent_finish");
}

}  // extern "C"

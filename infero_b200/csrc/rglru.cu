// A gated linear recurrence over channels (the recurrent block of Griffin: De, Smith et al., "Griffin: Mixing Gated
// Linear Recurrences with Local Attention for Efficient Language Models"), between the layer's input product and its
// output product.  The input product gives, per token, a gate branch y and a recurrent branch x, both C wide (32-bit,
// biases added).  Then, per channel c of request e:
//
//   u_t   = sum_j conv[c, j] * x_(t - (taps - 1 - j)) + conv_b[c]         (zeros before the sequence)
//   r_t   = sigmoid(Ra[b] u_t,b + ra_b),  i_t = sigmoid(Ri[b] u_t,b + ri_b)  (b: the block of C / blocks channels c is in)
//   log a = -slope * r_t * softplus(lam[c]);   a = exp(log a)
//   S_t   = a S_(t-1) + sqrt(1 - a^2) * i_t * u_t                          (S = 0 before the sequence)
//   out_t = S_t * gelu_tanh(y_t) * scale
//
// all in 32-bit; 1 - a^2 is formed as -expm1(2 log a), which keeps its digits where a is close to 1.  What a request
// carries from step to step lives in its state slot, float32 [taps, C]: rows 0 .. taps-2 the last inputs x of the
// convolution (oldest first), row taps-1 the state S.
//
// Three launches: rglru_conv (u for every token of the step, from the step's rows and the request's tail; optionally a
// bf16 copy of u for a tensor-core gate product), the gate products (rglru_gates: 32-bit tiles with one fused
// multiply-add per k in ascending k, so a token's gates do not depend on the batch; or, for long bf16 portions, the
// engine's tensor-core product block by block) and rglru_scan.  The gate products are laid out block by block:
// gates[t, b, 0, :] the products of Ra[b], gates[t, b, 1, :] those of Ri[b] (each C / blocks wide).
//
// rglru_scan: a block takes 32 channels of one request; its warps cut the request's new tokens into as many segments.
// S_t = a_t S_(t-1) + b_t is linear in S, so each warp first runs its segment from S = 0 and leaves (product of a, end
// state); the segments before a warp's own are then folded in order to give its start state, and a second pass writes
// the outputs.  Single tokens and short portions run as one segment, in order.  The last warp writes the new S, the
// first the new tail.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanhf_(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

constexpr int MAX_TAPS = 16;

__global__ void rglru_conv_kernel(const float* __restrict__ proj, int proj_stride, int x_off, const float* __restrict__ conv_w,
                                  const float* __restrict__ conv_b, int taps, const float* __restrict__ state,
                                  const int* __restrict__ tok_entry, const int* __restrict__ entry_q_start,
                                  const int* __restrict__ entry_slot, float* __restrict__ u, bf16* __restrict__ u16,
                                  int n_tokens, int C) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * C) return;
    const int t = (int)(idx / C), c = (int)(idx % C);
    const int e = tok_entry[t];
    const int local = t - entry_q_start[e];                  // index of the token within its request's portion
    const float* tail = state + (size_t)entry_slot[e] * taps * C;
    float acc = conv_b ? conv_b[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                        // how many tokens before this one
        float xv;
        if (back <= local) xv = proj[(size_t)(t - back) * proj_stride + x_off + c];
        else xv = tail[(size_t)(taps - 1 - (back - local)) * C + c];    // tail row taps-2 is the token just before the portion
        acc = fmaf(conv_w[(size_t)c * taps + j], xv, acc);
    }
    u[(size_t)t * C + c] = acc;
    if (u16) u16[(size_t)t * C + c] = __float2bfloat16_rn(acc);
}

constexpr int BM = 64, BN = 64, BK = 16;

// out[t, b * 2 bs + n] = sum_k u[t, b * bs + k] * W[b, n, k],  W [blocks, 2 bs, bs]: the rows of Ra[b], then those of Ri[b]
template <typename TW>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const float* __restrict__ u, const TW* __restrict__ wg, float* __restrict__ out, int M, int C, int bs) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
    const int b = blockIdx.z, N = 2 * bs;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const float* A = u + (size_t)b * bs;
    const TW* W = wg + (size_t)b * N * bs;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < bs; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < bs) ? A[(size_t)gm * C + gk] : 0.f;
            Ws[kk][r] = (gn < N && gk < bs) ? to_f32(W[(size_t)gn * bs + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) out[(size_t)gm * 2 * C + (size_t)b * N + gn] = acc[i][j];
        }
    }
}

constexpr int MAX_SEGS = 16;

template <typename T>
__global__ void __launch_bounds__(32 * MAX_SEGS)
rglru_scan_kernel(const float* __restrict__ proj, int proj_stride, int y_off, int x_off, const float* __restrict__ u,
                  const float* __restrict__ gates, const float* __restrict__ ra_b, const float* __restrict__ ri_b,
                  const float* __restrict__ lam, float slope, int taps, float* __restrict__ state,
                  const int* __restrict__ entry_q_start, const int* __restrict__ entry_q_len,
                  const int* __restrict__ entry_slot, T* __restrict__ out, int out_stride, int C, int bs, float scale) {
    __shared__ float As[MAX_SEGS][32], Bs[MAX_SEGS][32];
    const int tx = threadIdx.x, w = threadIdx.y, segs = blockDim.y;
    const int c = blockIdx.x * 32 + tx;
    const bool live = c < C;
    const int e = blockIdx.y;
    const int t0 = entry_q_start[e], n = entry_q_len[e];
    if (n <= 0) return;                                      // (the whole block: n is the request's)
    float* st = state + (size_t)entry_slot[e] * taps * C;
    // segments of about 32 tokens, as many as the request's own portion asks for (what else is in the step does not
    // change how a request is cut); warps beyond that have nothing to do but pass the state on
    const int eff = min(segs, max(1, (n + 31) / 32));
    const int seg = (n + eff - 1) / eff;
    const int k0 = min(n, w * seg), k1 = min(n, k0 + seg);
    float S = 0.f, sp = 0.f, ba = 0.f, bi = 0.f;
    size_t gcol = 0;
    if (live) {
        S = st[(size_t)(taps - 1) * C + c];
        sp = slope * softplusf_(lam[c]);
        ba = ra_b[c], bi = ri_b[c];
        gcol = (size_t)(c / bs) * 2 * bs + (c % bs);
    }
    // a_t and b_t of token k: S_t = a_t S_(t-1) + b_t
    auto step = [&](int k, float& a, float& b) {
        const size_t t = (size_t)(t0 + k);
        const float uv = u[t * C + c];
        const float r = sigmoidf_(gates[t * 2 * C + gcol] + ba);
        const float i = sigmoidf_(gates[t * 2 * C + gcol + bs] + bi);
        const float log_a = -sp * r;
        a = expf(log_a);
        b = sqrtf(-expm1f(2.0f * log_a)) * (i * uv);
    };
    if (segs > 1) {
        float A = 1.f, B = 0.f;
        if (live)
            for (int k = k0; k < k1; ++k) {
                float a, b;
                step(k, a, b);
                B = fmaf(a, B, b);
                A *= a;
            }
        As[w][tx] = A, Bs[w][tx] = B;
        __syncthreads();
        for (int j = 0; j < w; ++j) S = fmaf(As[j][tx], S, Bs[j][tx]);
    }
    if (!live) return;
    for (int k = k0; k < k1; ++k) {
        float a, b;
        step(k, a, b);
        S = fmaf(a, S, b);
        const size_t t = (size_t)(t0 + k);
        const float y = gelu_tanhf_(proj[t * proj_stride + y_off + c]);
        out[t * out_stride + c] = from_f32<T>(S * y * scale);
    }
    if (w == segs - 1) st[(size_t)(taps - 1) * C + c] = S;      // (an empty last segment holds the folded state)
    if (w == 0) {
        // the new tail: the last taps-1 inputs of (old tail, this portion), oldest first
        float keep[MAX_TAPS];
        for (int j = 0; j < taps - 1; ++j) {
            const int back = taps - 1 - j;                        // 1 = the newest input
            keep[j] = back <= n ? proj[(size_t)(t0 + n - back) * proj_stride + x_off + c]
                                : st[(size_t)(taps - 1 - (back - n)) * C + c];
        }
        for (int j = 0; j < taps - 1; ++j) st[(size_t)j * C + c] = keep[j];
    }
}

}  // namespace

extern "C" {

int infero_rglru_conv(const float* proj, int proj_stride, int x_off, const float* conv_w, const float* conv_b, int taps,
                      const float* state, const int* tok_entry, const int* entry_q_start, const int* entry_slot, float* u,
                      void* u_bf16, int n_tokens, int C, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "rglru: %d taps outside 1..%d", taps, MAX_TAPS);
    const long long total = (long long)n_tokens * C;
    rglru_conv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(proj, proj_stride, x_off, conv_w, conv_b, taps, state,
                                                                          tok_entry, entry_q_start, entry_slot, u, (bf16*)u_bf16, n_tokens, C);
    return infero_check_launch("rglru_conv");
}

int infero_rglru_gates(const float* u, const void* wg, int w_dtype, float* out, int n_tokens, int C, int blocks,
                       cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(blocks >= 1 && C % blocks == 0, "rglru: %d channels in %d blocks", C, blocks);
    const int bs = C / blocks, tiles_n = (2 * bs + BN - 1) / BN;
    INFERO_REQUIRE((n_tokens + BM - 1) / BM <= 65535 && blocks <= 65535, "rglru: grid too large");
    dim3 grid(tiles_n, (n_tokens + BM - 1) / BM, blocks);
    if (w_dtype == INFERO_F32)
        rglru_gates_kernel<float><<<grid, 256, 0, stream>>>(u, (const float*)wg, out, n_tokens, C, bs);
    else
        rglru_gates_kernel<bf16><<<grid, 256, 0, stream>>>(u, (const bf16*)wg, out, n_tokens, C, bs);
    return infero_check_launch("rglru_gates");
}

int infero_rglru_scan(const float* proj, int proj_stride, int y_off, int x_off, const float* u, const float* gates,
                      const float* ra_b, const float* ri_b, const float* lam, float slope, int taps, float* state,
                      const int* entry_q_start, const int* entry_q_len, const int* entry_slot, void* out, int out_stride,
                      int out_dtype, int n_entries, int C, int blocks, int max_q_len, float scale, cudaStream_t stream) {
    if (n_entries == 0) return 0;
    INFERO_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "rglru: %d taps outside 1..%d", taps, MAX_TAPS);
    INFERO_REQUIRE(n_entries <= 65535, "rglru: %d requests in a step", n_entries);
    INFERO_REQUIRE(blocks >= 1 && C % blocks == 0, "rglru: %d channels in %d blocks", C, blocks);
    // enough warps for the longest portion of the step; each request uses as many as its own portion asks for
    int segs = (max_q_len + 31) / 32;
    segs = segs < 1 ? 1 : segs > MAX_SEGS ? MAX_SEGS : segs;
    dim3 grid((C + 31) / 32, n_entries), block(32, segs);
    if (out_dtype == INFERO_F32)
        rglru_scan_kernel<float><<<grid, block, 0, stream>>>(proj, proj_stride, y_off, x_off, u, gates, ra_b, ri_b, lam, slope, taps,
                                                             state, entry_q_start, entry_q_len, entry_slot, (float*)out,
                                                             out_stride, C, C / blocks, scale);
    else
        rglru_scan_kernel<bf16><<<grid, block, 0, stream>>>(proj, proj_stride, y_off, x_off, u, gates, ra_b, ri_b, lam, slope, taps,
                                                            state, entry_q_start, entry_q_len, entry_slot, (bf16*)out,
                                                            out_stride, C, C / blocks, scale);
    return infero_check_launch("rglru_scan");
}

}  // extern "C"

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
// With the tensor-core product the bf16 copy of u and the gates are laid out block-major ([blocks, rows, ...], rows padded
// to the product's tile) so that one grouped product does all blocks.  rglru_scan is described at the kernel.
#include "common.cuh"

namespace {

// (a correctly rounded reciprocal in place of the division: a few instructions instead of a dozen)
__device__ __forceinline__ float sigmoidf_(float z) { return __frcp_rn(1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
// 0.5 z (1 + tanh w) = z / (1 + exp(-2 w)), w = sqrt(2 / pi) (z + 0.044715 z^3)
__device__ __forceinline__ float gelu_tanhf_(float z) {
    const float w = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return z * __frcp_rn(1.0f + expf(-2.0f * w));
}

// Where the result is rounded to bf16, the hardware's approximate exponential, reciprocal and root (relative errors of
// about 1e-6) take the place of the correctly rounded sequences: a third of the scan's instructions.  32-bit results
// keep the exact forms.
template <bool FAST> __device__ __forceinline__ float sigmoid_(float z) {
    if constexpr (FAST) return __fdividef(1.0f, 1.0f + __expf(-z));
    else return sigmoidf_(z);
}
template <bool FAST> __device__ __forceinline__ float gelu_tanh_(float z) {
    if constexpr (FAST) {
        const float w = 0.7978845608028654f * (z + 0.044715f * z * z * z);
        return z * __fdividef(1.0f, 1.0f + __expf(-2.0f * w));
    } else return gelu_tanhf_(z);
}
// exp(x) - 1 for x <= 0: the series where x is small (so that 1 - a^2 keeps its digits), else the exponential
template <bool FAST> __device__ __forceinline__ float expm1_(float x) {
    if constexpr (FAST) {
        const float p = x * (1.0f + x * (0.5f + x * (0.16666667f + x * (0.041666668f + x * 0.0083333338f))));
        return x > -0.0625f ? p : __expf(x) - 1.0f;
    } else return expm1f(x);
}
template <bool FAST> __device__ __forceinline__ float sqrt_(float x) {
    if constexpr (FAST) {
        float r;
        asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
        return r;
    } else return sqrtf(x);
}

constexpr int MAX_TAPS = 16;

__global__ void rglru_conv_kernel(const float* __restrict__ proj, int proj_stride, int x_off, const float* __restrict__ conv_w,
                                  const float* __restrict__ conv_b, int taps, const float* __restrict__ state,
                                  const int* __restrict__ tok_entry, const int* __restrict__ entry_q_start,
                                  const int* __restrict__ entry_slot, float* __restrict__ u, bf16* __restrict__ u16,
                                  int bs, long long u16_blk, int n_tokens, int C) {
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
        acc = fmaf(conv_w[(size_t)j * C + c], xv, acc);
    }
    u[(size_t)t * C + c] = acc;
    if (u16) u16[(size_t)(c / bs) * u16_blk + (size_t)t * bs + (c % bs)] = __float2bfloat16_rn(acc);
}

// The same for four neighbouring channels a thread (all offsets and C in multiples of four, 16-byte aligned rows).
__global__ void rglru_conv_vec4_kernel(const float* __restrict__ proj, int proj_stride, int x_off, const float* __restrict__ conv_w,
                                       const float* __restrict__ conv_b, int taps, const float* __restrict__ state,
                                       const int* __restrict__ tok_entry, const int* __restrict__ entry_q_start,
                                       const int* __restrict__ entry_slot, float* __restrict__ u, bf16* __restrict__ u16,
                                       int bs, long long u16_blk, int n_tokens, int C) {
    const int C4 = C / 4;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * C4) return;
    const int t = (int)(idx / C4), c = (int)(idx % C4) * 4;
    const int e = tok_entry[t];
    const int local = t - entry_q_start[e];
    const float* tail = state + (size_t)entry_slot[e] * taps * C;
    float4 acc = conv_b ? *reinterpret_cast<const float4*>(conv_b + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const float* src = back <= local ? proj + (size_t)(t - back) * proj_stride + x_off + c
                                         : tail + (size_t)(taps - 1 - (back - local)) * C + c;
        const float4 xv = *reinterpret_cast<const float4*>(src);
        const float4 wv = *reinterpret_cast<const float4*>(conv_w + (size_t)j * C + c);
        acc.x = fmaf(wv.x, xv.x, acc.x);
        acc.y = fmaf(wv.y, xv.y, acc.y);
        acc.z = fmaf(wv.z, xv.z, acc.z);
        acc.w = fmaf(wv.w, xv.w, acc.w);
    }
    *reinterpret_cast<float4*>(u + (size_t)t * C + c) = acc;
    if (u16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 pk;
        pk.x = *reinterpret_cast<unsigned*>(&lo);
        pk.y = *reinterpret_cast<unsigned*>(&hi);
        *reinterpret_cast<uint2*>(u16 + (size_t)(c / bs) * u16_blk + (size_t)t * bs + (c % bs)) = pk;
    }
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

// Steps of a few tokens with bf16 matrices: a warp per result column, its lanes along the contraction (eight
// weights a load), the step's tokens in registers; a tree of shuffles adds the lanes up.  Same layout of the results.
template <int MT>
__global__ void __launch_bounds__(256)
rglru_gates_skinny_kernel(const float* __restrict__ u, const bf16* __restrict__ wg, float* __restrict__ out, int M, int C, int bs) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= 2 * C) return;
    const int N = 2 * bs, b = warp / N, n = warp % N;
    const bf16* w = wg + ((size_t)b * N + n) * bs;
    const float* a = u + (size_t)b * bs;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    for (int k = lane * 8; k < bs; k += 256) {
        const uint4 raw = *reinterpret_cast<const uint4*>(w + k);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float wv[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p2[i]);
            wv[2 * i] = f.x, wv[2 * i + 1] = f.y;
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const float4 a0 = *reinterpret_cast<const float4*>(a + (size_t)m * C + k);
                const float4 a1 = *reinterpret_cast<const float4*>(a + (size_t)m * C + k + 4);
                float s = acc[m];
                s = fmaf(a0.x, wv[0], s), s = fmaf(a0.y, wv[1], s), s = fmaf(a0.z, wv[2], s), s = fmaf(a0.w, wv[3], s);
                s = fmaf(a1.x, wv[4], s), s = fmaf(a1.y, wv[5], s), s = fmaf(a1.z, wv[6], s), s = fmaf(a1.w, wv[7], s);
                acc[m] = s;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        float s = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0 && m < M) out[(size_t)m * 2 * C + (size_t)b * N + n] = s;
    }
}

constexpr int SEG = 16;              // tokens of a segment

// A warp holds CH channels times 32 / CH segments; a block of W warps W * 32 / CH segments of SEG tokens: a stretch.  A
// request's new tokens are worked through stretch by stretch.  S_t = a_t S_(t-1) + b_t is linear in S, so every thread
// first runs its segment from S = 0, keeps (a_t, b_t) in shared memory and leaves (product of a, end value); the segments
// before a thread's own are folded in order from the stretch's start state, and the second pass runs the segment again
// from there, from the kept pairs, and writes the outputs.  The thread that ran the stretch's last segment hands its
// end state to the next stretch; the one that ran the request's last token writes the new S.  How a request is cut
// depends on its own length alone (segments of SEG tokens from its first new token), and the fold is in order, so
// neither the width of a block nor what else is in the step changes a bit of the result.
// gates: the products of token t, block b at gates + t * g_tok + b * g_blk: Ra's bs, then Ri's bs.
template <typename T, int CH>
__global__ void __launch_bounds__(256, 2)
rglru_scan_kernel(const float* __restrict__ proj, int proj_stride, int y_off, int x_off, const float* __restrict__ u,
                  const float* __restrict__ gates, long long g_tok, long long g_blk, const float* __restrict__ ra_b,
                  const float* __restrict__ ri_b, const float* __restrict__ lam, float slope, int taps,
                  float* __restrict__ state, const int* __restrict__ entry_q_start, const int* __restrict__ entry_q_len,
                  const int* __restrict__ entry_slot, T* __restrict__ out, int out_stride, int C, int bs, float scale) {
    constexpr int SUB = 32 / CH;
    constexpr bool FAST = sizeof(T) == 2;
    extern __shared__ float2 scan_smem[];
    const int threads = blockDim.x, tid = threadIdx.x;
    const int nseg = (threads / 32) * SUB;
    float2* ab = scan_smem;                                  // [SEG][threads]
    float2* fold = scan_smem + (size_t)SEG * threads;        // [nseg][CH]
    float* carry = reinterpret_cast<float*>(fold + (size_t)nseg * CH);   // [CH]
    const int lane = tid & 31, ch = lane % CH, segi = (tid >> 5) * SUB + lane / CH;
    const int c = blockIdx.x * CH + ch;
    const bool live = c < C;
    const int e = blockIdx.y;
    const int t0 = entry_q_start[e], n = entry_q_len[e];
    if (n <= 0) return;                                      // (the whole block: n is the request's)
    float* st = state + (size_t)entry_slot[e] * taps * C;
    float sp = 0.f, ba = 0.f, bi = 0.f;
    const float* gp = gates;
    if (live) {
        sp = slope * softplusf_(lam[c]);
        ba = ra_b[c], bi = ri_b[c];
        gp = gates + (size_t)(c / bs) * g_blk + (c % bs);
        if (segi == 0) carry[ch] = st[(size_t)(taps - 1) * C + c];
    }
    for (int base = 0; base < n; base += nseg * SEG) {
        const int k0 = min(n, base + segi * SEG), k1 = min(n, k0 + SEG);
        float A = 1.f, B = 0.f;
        if (live && k0 < k1) {
            // all of the segment's loads first, so that they are in flight together
            float uv[SEG], gr[SEG], gi[SEG];
#pragma unroll
            for (int j = 0; j < SEG; ++j) {
                const size_t t = (size_t)(t0 + min(k0 + j, k1 - 1));
                uv[j] = u[t * C + c];
                gr[j] = gp[t * g_tok];
                gi[j] = gp[t * g_tok + bs];
            }
#pragma unroll
            for (int j = 0; j < SEG; ++j) {
                if (k0 + j < k1) {
                    const float r = sigmoid_<FAST>(gr[j] + ba);
                    const float i = sigmoid_<FAST>(gi[j] + bi);
                    // a = exp(log a) = 1 + e with e = expm1(log a); 1 - a^2 = -e (2 + e) keeps its digits where a is close to 1
                    const float e = expm1_<FAST>(-sp * r);
                    const float a = 1.0f + e;
                    const float b = sqrt_<FAST>(-e * (2.0f + e)) * (i * uv[j]);
                    ab[(size_t)j * threads + tid] = make_float2(a, b);
                    B = fmaf(a, B, b);
                    A *= a;
                }
            }
        }
        fold[segi * CH + ch] = make_float2(A, B);
        __syncthreads();
        float S = carry[ch];
        for (int j = 0; j < segi; ++j) {
            const float2 f = fold[j * CH + ch];
            S = fmaf(f.x, S, f.y);
        }
        __syncthreads();                                     // (every thread has read the stretch's start state)
        if (live) {
            if (k0 < k1) {
                float yv[SEG];
#pragma unroll
                for (int j = 0; j < SEG; ++j) yv[j] = proj[(size_t)(t0 + min(k0 + j, k1 - 1)) * proj_stride + y_off + c];
#pragma unroll
                for (int j = 0; j < SEG; ++j) {
                    if (k0 + j < k1) {
                        const float2 f = ab[(size_t)j * threads + tid];
                        S = fmaf(f.x, S, f.y);
                        out[(size_t)(t0 + k0 + j) * out_stride + c] = from_f32<T>(S * gelu_tanh_<FAST>(yv[j]) * scale);
                    }
                }
            }
            if (k0 < n && k1 == n) st[(size_t)(taps - 1) * C + c] = S;          // ran the request's last token
            else if (segi == nseg - 1) carry[ch] = S;                              // ran the stretch's last segment
        }
        __syncthreads();
    }
    if (live && segi == 0) {
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

// Steps in which every request brings one token, bf16 matrices, blocks of up to 256 channels: convolution, gate
// products and the state's update in one launch.  A thread block owns one block of channels of one request (so nothing
// it reads of the state is written by another): u of the block's channels into shared memory, a warp per gate row
// (eight weights a load, lanes along the contraction), then a thread per channel updates S, writes the result and
// shifts the convolution's tail.
template <typename T>
__global__ void __launch_bounds__(256)
rglru_step_kernel(const float* __restrict__ proj, int proj_stride, int y_off, int x_off, const float* __restrict__ conv_wt,
                  const float* __restrict__ conv_b, int taps, const bf16* __restrict__ wg, const float* __restrict__ ra_b,
                  const float* __restrict__ ri_b, const float* __restrict__ lam, float slope, float* __restrict__ state,
                  const int* __restrict__ entry_q_start, const int* __restrict__ entry_q_len,
                  const int* __restrict__ entry_slot, T* __restrict__ out, int out_stride, int C, int bs, float scale) {
    constexpr bool FAST = sizeof(T) == 2;
    __shared__ __align__(16) float us[256];
    __shared__ float xs[256], gs[512];
    const int b = blockIdx.x, e = blockIdx.y, tid = threadIdx.x;
    if (entry_q_len[e] <= 0) return;
    const size_t t = (size_t)entry_q_start[e];
    float* st = state + (size_t)entry_slot[e] * taps * C;
    const int c = b * bs + tid;
    if (tid < bs) {
        // tail row j holds the input taps-1-j tokens back, which tap j multiplies; the last tap takes this token's
        const float x = proj[t * proj_stride + x_off + c];
        float acc = conv_b ? conv_b[c] : 0.f;
        for (int j = 0; j < taps - 1; ++j) acc = fmaf(conv_wt[(size_t)j * C + c], st[(size_t)j * C + c], acc);
        acc = fmaf(conv_wt[(size_t)(taps - 1) * C + c], x, acc);
        us[tid] = acc, xs[tid] = x;
    }
    __syncthreads();
    // a row of the gate matrices takes bs / 8 lanes (a power of two of them): a warp works on 32 / lanes rows at a time,
    // four such groups per turn with their loads issued together
    const int warp = tid >> 5, lane = tid & 31;
    int lanes = 1;
    while (lanes * 8 < bs) lanes <<= 1;
    const int per = 32 / lanes, sub = lane / lanes, k = (lane % lanes) * 8;
    const bool in = k < bs;
    const bf16* W = wg + (size_t)b * 2 * bs * bs;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    if (in) a0 = *reinterpret_cast<const float4*>(us + k), a1 = *reinterpret_cast<const float4*>(us + k + 4);
    for (int n0 = warp * per * 4; n0 < 2 * bs; n0 += 8 * per * 4) {
        uint4 raw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int n = n0 + q * per + sub;
            raw[q] = (in && n < 2 * bs) ? *reinterpret_cast<const uint4*>(W + (size_t)n * bs + k) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int n = n0 + q * per + sub;
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw[q]);
            const float2 w0 = __bfloat1622float2(p2[0]), w1 = __bfloat1622float2(p2[1]);
            const float2 w2 = __bfloat1622float2(p2[2]), w3 = __bfloat1622float2(p2[3]);
            float s = 0.f;
            s = fmaf(a0.x, w0.x, s), s = fmaf(a0.y, w0.y, s), s = fmaf(a0.z, w1.x, s), s = fmaf(a0.w, w1.y, s);
            s = fmaf(a1.x, w2.x, s), s = fmaf(a1.y, w2.y, s), s = fmaf(a1.z, w3.x, s), s = fmaf(a1.w, w3.y, s);
            for (int o = lanes >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane % lanes == 0 && n < 2 * bs) gs[n] = s;
        }
    }
    __syncthreads();
    if (tid < bs) {
        const float r = sigmoid_<FAST>(gs[tid] + ra_b[c]);
        const float i = sigmoid_<FAST>(gs[bs + tid] + ri_b[c]);
        const float e1 = expm1_<FAST>(-slope * softplusf_(lam[c]) * r);
        const float a = 1.0f + e1;
        const float S = fmaf(a, st[(size_t)(taps - 1) * C + c], sqrt_<FAST>(-e1 * (2.0f + e1)) * (i * us[tid]));
        st[(size_t)(taps - 1) * C + c] = S;
        out[t * out_stride + c] = from_f32<T>(S * gelu_tanh_<FAST>(proj[t * proj_stride + y_off + c]) * scale);
        for (int j = 0; j + 2 < taps; ++j) st[(size_t)j * C + c] = st[(size_t)(j + 1) * C + c];
        if (taps >= 2) st[(size_t)(taps - 2) * C + c] = xs[tid];
    }
}

}  // namespace

extern "C" {

// u_bf16 (optional): a bf16 copy of u laid out block by block, [blocks, rows_per_block, C / blocks], for a grouped
// tensor-core product of the gates.
int infero_rglru_conv(const float* proj, int proj_stride, int x_off, const float* conv_w, const float* conv_b, int taps,
                      const float* state, const int* tok_entry, const int* entry_q_start, const int* entry_slot, float* u,
                      void* u_bf16, int blocks, long long rows_per_block, int n_tokens, int C, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "rglru: %d taps outside 1..%d", taps, MAX_TAPS);
    INFERO_REQUIRE(!u_bf16 || (blocks >= 1 && C % blocks == 0 && rows_per_block >= n_tokens), "rglru: bad layout of the bf16 copy");
    const long long total = (long long)n_tokens * C;
    const int bs = u_bf16 ? C / blocks : C;
    const bool vec4 = C % 4 == 0 && bs % 4 == 0 && proj_stride % 4 == 0 && x_off % 4 == 0 && (uintptr_t)proj % 16 == 0 &&
                      (uintptr_t)u % 16 == 0 && (uintptr_t)state % 16 == 0 && (uintptr_t)conv_w % 16 == 0 && (!conv_b || (uintptr_t)conv_b % 16 == 0) &&
                      (!u_bf16 || (uintptr_t)u_bf16 % 8 == 0);
    if (vec4)
        rglru_conv_vec4_kernel<<<(unsigned)((total / 4 + 255) / 256), 256, 0, stream>>>(proj, proj_stride, x_off, conv_w, conv_b, taps,
                                                                                       state, tok_entry, entry_q_start, entry_slot, u,
                                                                                       (bf16*)u_bf16, bs, rows_per_block * bs, n_tokens, C);
    else
        rglru_conv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(proj, proj_stride, x_off, conv_w, conv_b, taps, state,
                                                                              tok_entry, entry_q_start, entry_slot, u, (bf16*)u_bf16,
                                                                              bs, rows_per_block * bs, n_tokens, C);
    return infero_check_launch("rglru_conv");
}

int infero_rglru_gates(const float* u, const void* wg, int w_dtype, float* out, int n_tokens, int C, int blocks,
                       cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(blocks >= 1 && C % blocks == 0, "rglru: %d channels in %d blocks", C, blocks);
    const int bs = C / blocks, tiles_n = (2 * bs + BN - 1) / BN;
    INFERO_REQUIRE((n_tokens + BM - 1) / BM <= 65535 && blocks <= 65535, "rglru: grid too large");
    dim3 grid(tiles_n, (n_tokens + BM - 1) / BM, blocks);
    if (w_dtype != INFERO_F32 && n_tokens <= 16 && bs % 8 == 0 && (uintptr_t)wg % 16 == 0 && (uintptr_t)u % 16 == 0) {
        const unsigned nb = (unsigned)((2ll * C * 32 + 255) / 256);
        if (n_tokens <= 4) rglru_gates_skinny_kernel<4><<<nb, 256, 0, stream>>>(u, (const bf16*)wg, out, n_tokens, C, bs);
        else if (n_tokens <= 8) rglru_gates_skinny_kernel<8><<<nb, 256, 0, stream>>>(u, (const bf16*)wg, out, n_tokens, C, bs);
        else rglru_gates_skinny_kernel<16><<<nb, 256, 0, stream>>>(u, (const bf16*)wg, out, n_tokens, C, bs);
        return infero_check_launch("rglru_gates_skinny");
    }
    if (w_dtype == INFERO_F32)
        rglru_gates_kernel<float><<<grid, 256, 0, stream>>>(u, (const float*)wg, out, n_tokens, C, bs);
    else
        rglru_gates_kernel<bf16><<<grid, 256, 0, stream>>>(u, (const bf16*)wg, out, n_tokens, C, bs);
    return infero_check_launch("rglru_gates");
}

// gates: token t's products for block b start at gates + t * g_tok + b * g_blk (floats): Ra[b]'s, then Ri[b]'s.
// (token-major from rglru_gates: g_tok = 2 C, g_blk = 2 C / blocks; block-major from a grouped product over
// [blocks, rows, C / blocks]: g_tok = 2 C / blocks, g_blk = rows * 2 C / blocks.)
int infero_rglru_scan(const float* proj, int proj_stride, int y_off, int x_off, const float* u, const float* gates,
                      long long g_tok, long long g_blk, const float* ra_b, const float* ri_b, const float* lam, float slope,
                      int taps, float* state, const int* entry_q_start, const int* entry_q_len, const int* entry_slot,
                      void* out, int out_stride, int out_dtype, int n_entries, int C, int blocks, int max_q_len, float scale,
                      cudaStream_t stream) {
    if (n_entries == 0) return 0;
    INFERO_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "rglru: %d taps outside 1..%d", taps, MAX_TAPS);
    INFERO_REQUIRE(n_entries <= 65535, "rglru: %d requests in a step", n_entries);
    INFERO_REQUIRE(blocks >= 1 && C % blocks == 0, "rglru: %d channels in %d blocks", C, blocks);
    const int bs = C / blocks;
    // steps of short portions: a warp of 32 channels per segment, as many warps as the longest portion has segments (two
    // at most); steps with long portions: 8 channels times 4 segments a warp, 8 warps, two blocks a multiprocessor, so that
    // one block's loads overlap the other's arithmetic
    const bool wide = max_q_len > 2 * SEG;
    const int ch = wide ? 8 : 32;
    const int warps = wide ? 8 : (max_q_len > SEG ? 2 : 1);
    const int threads = 32 * warps, nseg = warps * (32 / ch);
    const size_t smem = (size_t)SEG * threads * sizeof(float2) + (size_t)nseg * ch * sizeof(float2) + ch * sizeof(float);
    dim3 grid((C + ch - 1) / ch, n_entries);
#define LAUNCH(T, CH)                                                                                                    \
    do {                                                                                                                 \
        auto k = rglru_scan_kernel<T, CH>;                                                                               \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        k<<<grid, threads, smem, stream>>>(proj, proj_stride, y_off, x_off, u, gates, g_tok, g_blk, ra_b, ri_b, lam,      \
                                           slope, taps, state, entry_q_start, entry_q_len, entry_slot, (T*)out,          \
                                           out_stride, C, bs, scale);                                                    \
    } while (0)
    if (out_dtype == INFERO_F32) {
        if (wide) LAUNCH(float, 8);
        else LAUNCH(float, 32);
    } else {
        if (wide) LAUNCH(bf16, 8);
        else LAUNCH(bf16, 32);
    }
#undef LAUNCH
    return infero_check_launch("rglru_scan");
}

// The whole recurrence of a step of single tokens in one launch (bf16 gate matrices, blocks of 8 .. 256 channels in
// multiples of 8); conv_wt tap-major [taps, C].  Returns 2 without launching where the sizes do not fit.
int infero_rglru_step(const float* proj, int proj_stride, int y_off, int x_off, const float* conv_wt, const float* conv_b,
                      int taps, const void* wg, const float* ra_b, const float* ri_b, const float* lam, float slope,
                      float* state, const int* entry_q_start, const int* entry_q_len, const int* entry_slot, void* out,
                      int out_stride, int out_dtype, int n_entries, int C, int blocks, float scale, cudaStream_t stream) {
    if (n_entries == 0) return 0;
    INFERO_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "rglru: %d taps outside 1..%d", taps, MAX_TAPS);
    INFERO_REQUIRE(blocks >= 1 && C % blocks == 0, "rglru: %d channels in %d blocks", C, blocks);
    const int bs = C / blocks;
    if (bs > 256 || bs % 8 || (uintptr_t)wg % 16 || n_entries > 65535) return 2;
    dim3 grid(blocks, n_entries);
    if (out_dtype == INFERO_F32)
        rglru_step_kernel<float><<<grid, 256, 0, stream>>>(proj, proj_stride, y_off, x_off, conv_wt, conv_b, taps, (const bf16*)wg, ra_b,
                                                           ri_b, lam, slope, state, entry_q_start, entry_q_len, entry_slot,
                                                           (float*)out, out_stride, C, bs, scale);
    else
        rglru_step_kernel<bf16><<<grid, 256, 0, stream>>>(proj, proj_stride, y_off, x_off, conv_wt, conv_b, taps, (const bf16*)wg, ra_b,
                                                          ri_b, lam, slope, state, entry_q_start, entry_q_len, entry_slot,
                                                          (bf16*)out, out_stride, C, bs, scale);
    return infero_check_launch("rglru_step");
}

}  // extern "C"

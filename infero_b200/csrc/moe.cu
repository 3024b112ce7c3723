// Mixture of experts: routing, and the experts of few tokens.
//
// select: from the router's logits z = Wr h (a product with 32-bit sums, made by the caller), per token the `top`
//   largest (lowest index wins a tie), their weights = softmax over the chosen logits only; optionally the gate of a
//   shared expert, the sigmoid of one more column of that product.  One warp per token.
// experts of few tokens (a weight-streaming path; every (token, choice) reads its expert's rows):
//   up:   act[t, c, j] = glu(Wg_e[j] . h_t, Wu_e[j] . h_t),  e = choice c of token t; one warp per j; glu is one of
//         the gated activations of common.cuh (silu(g) * u, or its clamped form)
//   down: y[t, i] = sum_c weight[t, c] * (Wd_e[i] . act[t, c]) (+ gate_t * shared[t, i]); one warp per i,
//         choices added in ascending c, so a token's result does not depend on the batch.
// Expert weights are stacked: gate_up [E, 2 ff, d] with rows alternating gate_j, up_j; down [E, d, ff].
//
// select by scores: every expert's score is the sigmoid of its logit; the `top` largest scores are chosen (lowest index
//   wins a tie); the weights are the chosen scores, divided by their sum where asked.
// ungated experts (up [E, ff, d]): act[t, c, j] = f(w * (Wu_e[j] . h_t)) with f the squared relu and w the pair's weight
//   where the weight multiplies what the expert reads (then the down stage adds the choices up unweighted), else 1.
#include "common.cuh"
#include <math_constants.h>

namespace {

constexpr int RWARPS = 4;
constexpr int MAX_E = 512;
constexpr int MAX_TOP = 32;

__device__ __forceinline__ float warp_dot(const float* __restrict__ a, const float* __restrict__ b, int n, int lane) {
    float s = 0.f;
    for (int i = lane; i < n; i += 32) s = fmaf(a[i], b[i], s);
    return warp_sum(s);
}
// bf16 rows that start on 16-byte boundaries and hold a multiple of 8 elements are read 16 bytes per lane
__device__ __forceinline__ float warp_dot(const bf16* __restrict__ a, const bf16* __restrict__ b, int n, int lane) {
    float s = 0.f;
    if ((n & 7) == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0) {
        for (int i = lane * 8; i < n; i += 256) {
            const uint4 ua = *reinterpret_cast<const uint4*>(a + i), ub = *reinterpret_cast<const uint4*>(b + i);
            const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ua);
            const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __bfloat1622float2(pa[j]), fb = __bfloat1622float2(pb[j]);
                s = fmaf(fa.x, fb.x, s);
                s = fmaf(fa.y, fb.y, s);
            }
        }
    } else {
        for (int i = lane; i < n; i += 32) s = fmaf(__bfloat162float(a[i]), __bfloat162float(b[i]), s);
    }
    return warp_sum(s);
}

// logits float32 [tokens, stride]: columns 0..E-1 are the router's logits; column gate_col (if >= 0) is the logit of
// the shared expert's gate.
__global__ void __launch_bounds__(RWARPS * 32)
moe_select_kernel(const float* __restrict__ logits, int stride, int gate_col, int* __restrict__ top_idx,
                  float* __restrict__ top_w, float* __restrict__ gate_out, int n_tokens, int E, int top) {
    __shared__ float z[RWARPS][MAX_E];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * RWARPS + warp;
    if (t >= n_tokens) return;
    const float* zr = logits + (size_t)t * stride;
    for (int e = lane; e < E; e += 32) z[warp][e] = zr[e];
    if (gate_col >= 0 && lane == 0) gate_out[t] = 1.0f / (1.0f + expf(-zr[gate_col]));
    __syncwarp();
    float first = 0.f, mine = 0.f, sum = 0.f;
    int mine_e = 0;
    for (int c = 0; c < top; ++c) {
        float best = -CUDART_INF_F;
        int be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[warp][e];
            if (v > best) best = v, be = e;               // ascending e: the lowest index of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > best || (ov == best && oe < be)) best = ov, be = oe;
        }
        if (c == 0) first = best;
        const float p = expf(best - first);
        sum += p;
        if (lane == c) mine = p, mine_e = be;
        __syncwarp();
        if (lane == 0) z[warp][be] = -CUDART_INF_F;
        __syncwarp();
    }
    if (lane < top) {
        top_idx[(size_t)t * top + lane] = mine_e;
        top_w[(size_t)t * top + lane] = mine / sum;
    }
}

// Scores are sigmoid(logit); the `top` largest are chosen by score (ties: the lower index); weights are the scores,
// divided by the sum of the chosen ones where `renorm`.  One warp per token.
__global__ void __launch_bounds__(RWARPS * 32)
moe_select_scored_kernel(const float* __restrict__ logits, int stride, int splits, long long split_stride,
                         int* __restrict__ top_idx, float* __restrict__ top_w, int n_tokens, int E, int top, int renorm) {
    __shared__ float sc[RWARPS][MAX_E];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * RWARPS + warp;
    if (t >= n_tokens) return;
    const float* zr = logits + (size_t)t * stride;
    for (int e = lane; e < E; e += 32) {
        float z = zr[e];                              // the logits may come as split-K partial sums, added up in order
        for (int sp = 1; sp < splits; ++sp) z += zr[(size_t)sp * split_stride + e];
        sc[warp][e] = 1.0f / (1.0f + expf(-z));
    }
    __syncwarp();
    float mine = 0.f, sum = 0.f;
    int mine_e = 0;
    for (int c = 0; c < top; ++c) {
        float best = -CUDART_INF_F;
        int be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = sc[warp][e];
            if (v > best) best = v, be = e;               // ascending e: the lowest index of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > best || (ov == best && oe < be)) best = ov, be = oe;
        }
        if (be == 0x7fffffff) be = 0, best = 0.f;         // nothing left to pick (scores that are no numbers)
        sum += best;
        if (lane == c) mine = best, mine_e = be;
        __syncwarp();
        if (lane == 0) sc[warp][be] = -CUDART_INF_F;
        __syncwarp();
    }
    if (lane < top) {
        top_idx[(size_t)t * top + lane] = mine_e;
        top_w[(size_t)t * top + lane] = renorm ? mine / (sum + 1e-20f) : mine;
    }
}

// Routing by a softmax over all experts with a per-expert correction of the choice and groups of experts:
//   s = softmax(z) over the E experts; pick score c_e = s_e + correction_e (correction may be null);
//   the experts form n_groups groups of E / n_groups neighbours, a group's score is its largest pick score, and only
//   experts of the `keep` best groups can be picked (ties: the lower group); the `top` largest pick scores among them
//   are chosen (ties: the lower expert); weights = s of the chosen / (their sum + 1e-20).  One warp per token.
__global__ void __launch_bounds__(RWARPS * 32)
moe_select_grouped_kernel(const float* __restrict__ logits, int stride, const float* __restrict__ correction,
                          int* __restrict__ top_idx, float* __restrict__ top_w, int n_tokens, int E, int top, int n_groups,
                          int keep) {
    __shared__ float sc[RWARPS][MAX_E];          // softmax scores
    __shared__ float pk[RWARPS][MAX_E];          // pick scores (minus infinity once taken or shut out)
    __shared__ float gs[RWARPS][MAX_E];          // group scores
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * RWARPS + warp;
    if (t >= n_tokens) return;
    const float* zr = logits + (size_t)t * stride;
    float mx = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float p = expf(zr[e] - mx);
        sc[warp][e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
        const float s = sc[warp][e] / sum;
        sc[warp][e] = s;
        pk[warp][e] = s + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float b = -CUDART_INF_F;
            for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, pk[warp][e]);
            gs[warp][g] = b;
        }
        __syncwarp();
        // a group is kept if fewer than `keep` groups are better (larger score, or equal score and lower index)
        for (int g = lane; g < n_groups; g += 32) {
            const float mine = gs[warp][g];
            int better = 0;
            for (int o = 0; o < n_groups; ++o) {
                const float v = gs[warp][o];
                better += (v > mine || (v == mine && o < g)) ? 1 : 0;
            }
            if (better >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) pk[warp][e] = -CUDART_INF_F;
        }
        __syncwarp();
    }
    float mine_s = 0.f, total = 0.f;
    int mine_e = 0;
    for (int c = 0; c < top; ++c) {
        float best = -CUDART_INF_F;
        int be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = pk[warp][e];
            if (v > best) best = v, be = e;               // ascending e: the lowest index of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > best || (ov == best && oe < be)) best = ov, be = oe;
        }
        if (be == 0x7fffffff) be = 0;                     // nothing left to pick (scores that are no numbers)
        const float s = sc[warp][be];
        total += s;
        if (lane == c) mine_s = s, mine_e = be;
        __syncwarp();
        if (lane == 0) pk[warp][be] = -CUDART_INF_F;
        __syncwarp();
    }
    if (lane < top) {
        top_idx[(size_t)t * top + lane] = mine_e;
        top_w[(size_t)t * top + lane] = mine_s / (total + 1e-20f);
    }
}

constexpr int EWARPS = 8;

template <typename T>
__global__ void __launch_bounds__(EWARPS * 32)
moe_up_kernel(const T* __restrict__ h, int h_stride, const T* __restrict__ gate_up, const int* __restrict__ top_idx,
              T* __restrict__ act, int d, int ff, int top, int act_kind, float act_limit, float act_alpha) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.y;                              // token * top + choice
    const int t = item / top;
    const int j = blockIdx.x * EWARPS + warp;
    if (j >= ff) return;
    const int e = top_idx[item];
    const T* hr = h + (size_t)t * h_stride;
    const T* wg = gate_up + ((size_t)e * 2 * ff + 2 * j) * d;
    const float g = warp_dot(wg, hr, d, lane);
    const float u = warp_dot(wg + d, hr, d, lane);
    if (lane == 0) act[(size_t)item * ff + j] = from_f32<T>(glu_act(g, u, act_kind, act_limit, act_alpha));
}

// Ungated experts: up [E, ff, d]; in_w (or null) multiplies the product before the squared relu.
template <typename T>
__global__ void __launch_bounds__(EWARPS * 32)
moe_up_plain_kernel(const T* __restrict__ h, int h_stride, const T* __restrict__ up, const int* __restrict__ top_idx,
                    const float* __restrict__ in_w, T* __restrict__ act, int d, int ff, int top) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.y;                              // token * top + choice
    const int t = item / top;
    const int j = blockIdx.x * EWARPS + warp;
    if (j >= ff) return;
    const int e = top_idx[item];
    float v = warp_dot(up + ((size_t)e * ff + j) * d, h + (size_t)t * h_stride, d, lane);
    if (in_w) v *= in_w[item];
    v = fmaxf(v, 0.f);
    if (lane == 0) act[(size_t)item * ff + j] = from_f32<T>(v * v);
}

template <typename T>
__global__ void __launch_bounds__(EWARPS * 32)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ down, const int* __restrict__ top_idx,
                const float* __restrict__ top_w, const float* __restrict__ shared, const float* __restrict__ shared_gate,
                float* __restrict__ y, int d, int ff, int top, int shared_splits = 1, long long shared_stride = 0) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    const int i = blockIdx.x * EWARPS + warp;
    if (i >= d) return;
    float acc = 0.f;
    for (int c = 0; c < top; ++c) {
        const int e = top_idx[(size_t)t * top + c];
        const float v = warp_dot(down + ((size_t)e * d + i) * ff, act + ((size_t)t * top + c) * ff, ff, lane);
        acc = top_w ? fmaf(top_w[(size_t)t * top + c], v, acc) : acc + v;
    }
    if (lane == 0) {
        if (shared) {
            float sh = shared[(size_t)t * d + i];                 // (split-K partial sums of the shared expert: added up in order)
            for (int sp = 1; sp < shared_splits; ++sp) sh += shared[(size_t)sp * shared_stride + (size_t)t * d + i];
            acc = fmaf(shared_gate ? shared_gate[t] : 1.0f, sh, acc);
        }
        y[(size_t)t * d + i] = acc;
    }
}

}  // namespace

extern "C" {

int infero_moe_select(const float* logits, int stride, int gate_col, int* top_idx, float* top_w, float* gate_out,
                      int n_tokens, int E, int top, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(E >= 1 && E <= MAX_E && top >= 1 && top <= E && top <= MAX_TOP,
                   "moe select: %d experts (at most %d), top %d (at most %d)", E, MAX_E, top, MAX_TOP);
    moe_select_kernel<<<(n_tokens + RWARPS - 1) / RWARPS, RWARPS * 32, 0, stream>>>(logits, stride, gate_col, top_idx, top_w,
                                                                                  gate_out, n_tokens, E, top);
    return infero_check_launch("moe_select");
}

int infero_moe_select_grouped(const float* logits, int stride, const float* correction, int* top_idx, float* top_w,
                              int n_tokens, int E, int top, int n_groups, int keep, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(E >= 1 && E <= MAX_E && top >= 1 && top <= E && top <= MAX_TOP,
                   "moe select: %d experts (at most %d), top %d (at most %d)", E, MAX_E, top, MAX_TOP);
    INFERO_REQUIRE(n_groups >= 1 && E % n_groups == 0 && keep >= 1 && keep <= n_groups && (E / n_groups) * keep >= top,
                   "moe select: %d groups of %d experts, %d kept, cannot give %d choices", n_groups, E, keep, top);
    moe_select_grouped_kernel<<<(n_tokens + RWARPS - 1) / RWARPS, RWARPS * 32, 0, stream>>>(
        logits, stride, correction, top_idx, top_w, n_tokens, E, top, n_groups, keep);
    return infero_check_launch("moe_select_grouped");
}

// logits: float32 [splits][tokens, stride] (split_stride elements apart); the value is the sum over the splits.
int infero_moe_select_scored(const float* logits, int stride, int splits, long long split_stride, int* top_idx, float* top_w,
                             int n_tokens, int E, int top, int renorm, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(E >= 1 && E <= MAX_E && top >= 1 && top <= E && top <= MAX_TOP,
                   "moe select: %d experts (at most %d), top %d (at most %d)", E, MAX_E, top, MAX_TOP);
    INFERO_REQUIRE(splits >= 1, "moe select: %d splits", splits);
    moe_select_scored_kernel<<<(n_tokens + RWARPS - 1) / RWARPS, RWARPS * 32, 0, stream>>>(logits, stride, splits, split_stride,
                                                                                         top_idx, top_w, n_tokens, E, top, renorm);
    return infero_check_launch("moe_select_scored");
}

// Ungated experts with the squared relu: up [E, ff, d], down [E, d, ff].  weight_input: the pair's weight multiplies what
// the expert reads and the choices are added up as they are; else it multiplies the expert's result.
// shared: float32 [shared_splits][tokens, d] (shared_stride elements apart; the value is the sum over the splits) or null.
int infero_moe_experts_plain_streamed(const void* h, int h_stride, const void* up, const void* down, int dtype,
                                      const int* top_idx, const float* top_w, int weight_input, const float* shared,
                                      int shared_splits, long long shared_stride, void* act, float* y, int n_tokens, int d,
                                      int ff, int top, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(n_tokens * (long long)top <= 65535 && n_tokens <= 65535, "moe: %d tokens are too many for the streaming path", n_tokens);
    const dim3 gu((ff + EWARPS - 1) / EWARPS, n_tokens * top), gd((d + EWARPS - 1) / EWARPS, n_tokens);
    const float* in_w = weight_input ? top_w : nullptr;
    const float* out_w = weight_input ? nullptr : top_w;
    if (dtype == INFERO_F32) {
        moe_up_plain_kernel<float><<<gu, EWARPS * 32, 0, stream>>>((const float*)h, h_stride, (const float*)up, top_idx, in_w,
                                                                  (float*)act, d, ff, top);
        moe_down_kernel<float><<<gd, EWARPS * 32, 0, stream>>>((const float*)act, (const float*)down, top_idx, out_w, shared,
                                                              nullptr, y, d, ff, top, shared_splits, shared_stride);
    } else {
        moe_up_plain_kernel<bf16><<<gu, EWARPS * 32, 0, stream>>>((const bf16*)h, h_stride, (const bf16*)up, top_idx, in_w,
                                                                 (bf16*)act, d, ff, top);
        moe_down_kernel<bf16><<<gd, EWARPS * 32, 0, stream>>>((const bf16*)act, (const bf16*)down, top_idx, out_w, shared,
                                                             nullptr, y, d, ff, top, shared_splits, shared_stride);
    }
    return infero_check_launch("moe_experts_plain_streamed");
}

// act: [tokens * top, ff] of dtype (scratch); y float32 [tokens, d]; shared float32 [tokens, d] or null.
int infero_moe_experts_streamed(const void* h, int h_stride, const void* gate_up, const void* down, int dtype,
                                const int* top_idx, const float* top_w, const float* shared, const float* shared_gate,
                                void* act, float* y, int n_tokens, int d, int ff, int top, int act_kind, float act_limit,
                                float act_alpha, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(n_tokens * (long long)top <= 65535 && n_tokens <= 65535, "moe: %d tokens are too many for the streaming path", n_tokens);
    const dim3 gu((ff + EWARPS - 1) / EWARPS, n_tokens * top), gd((d + EWARPS - 1) / EWARPS, n_tokens);
    if (dtype == INFERO_F32) {
        moe_up_kernel<float><<<gu, EWARPS * 32, 0, stream>>>((const float*)h, h_stride, (const float*)gate_up, top_idx,
                                                            (float*)act, d, ff, top, act_kind, act_limit, act_alpha);
        moe_down_kernel<float><<<gd, EWARPS * 32, 0, stream>>>((const float*)act, (const float*)down, top_idx, top_w,
                                                              shared, shared_gate, y, d, ff, top);
    } else {
        moe_up_kernel<bf16><<<gu, EWARPS * 32, 0, stream>>>((const bf16*)h, h_stride, (const bf16*)gate_up, top_idx,
                                                           (bf16*)act, d, ff, top, act_kind, act_limit, act_alpha);
        moe_down_kernel<bf16><<<gd, EWARPS * 32, 0, stream>>>((const bf16*)act, (const bf16*)down, top_idx, top_w,
                                                             shared, shared_gate, y, d, ff, top);
    }
    return infero_check_launch("moe_experts_streamed");
}

}  // extern "C"

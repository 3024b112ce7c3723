// A selective state-space recurrence with one scalar decay per head (the state-space-duality form), for any batch of
// requests, each with its new tokens and the state its earlier tokens left.
//
// The layer's input product gives, per token, [z | x | B | C | dt]: z and x are heads * P wide, B and C groups * N wide,
// dt has one number per head.  The channels of [x | B | C] (CH of them) pass a causal convolution of `taps` taps over
// time (weights [CH, taps], the last tap is the current token's; zeros before the start of a sequence) with a bias, and
// silu.  With dt = softplus(dt + dt_bias_h) and a_h = exp(A_log_h), head h (group h / (heads / groups)) keeps S [N, P]:
//
//     S <- exp(-a_h dt) S + dt B x^T          y = S^T C + D_h x
//
// and the layer's result before its output product is  rms_g(y * silu(z)) * w, the RMS norm taken over each of
// `norm_groups` equal parts of the heads * P channels.
//
// A request's state slot is float32 [(taps - 1) * CH + heads * N * P]: the convolution's last taps - 1 inputs (oldest
// first), then S laid out [heads, N, P].  Everything here is 32-bit; the result of the norm is written in the step's
// element type.
//
// conv:  one thread per (token, channel); inputs before the step's first token come from the slot's tail.
// tail:  after conv, one thread per (request, channel) moves the tail on by the request's new tokens.
// scan:  a block per (request, head, block of P columns); a thread keeps 16 rows of one column of S in registers;
//        tokens are staged sixteen at a time in shared memory by asynchronous copies, the next sixteen arriving while
//        these are worked on; the products with C are added up over the row groups in a fixed order.  The tokens of a
//        request run in order, so the arithmetic of a token does not depend on how the prompt was cut or on the rest
//        of the batch beyond rounding.  A portion of 256 tokens and more is cut into chunks of 128 of the request's
//        own tokens that run side by side: pass 1 (every chunk from S = 0: its end state and the product of its
//        decays), a chain over the chunks (start states), pass 2 (the outputs from the start states).
// gated group norm: one block per (token, part).
#include "common.cuh"
#include <stdlib.h>

namespace {

constexpr int NPT = 16;            // rows of S a thread keeps
constexpr int TCH = 16;            // tokens staged at a time (two stages: the next one arrives while this one is worked on)
constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }
__device__ __forceinline__ void copy4_async(float* dst_smem, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy16_async(float* dst_smem, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copies_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

__global__ void ssd_conv_kernel(const float* __restrict__ proj, int proj_stride, int x_off, const float* __restrict__ conv_w,
                                const float* __restrict__ conv_b, int taps, const float* __restrict__ state,
                                long long state_stride, const int* __restrict__ tok_entry,
                                const int* __restrict__ entry_q_start, const int* __restrict__ entry_slot,
                                float* __restrict__ u, int n_tokens, int CH) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * CH) return;
    const int t = (int)(idx / CH), c = (int)(idx % CH);
    const int e = tok_entry[t];
    const int first = entry_q_start[e];
    const int i = t - first;
    const float* tail = state + (long long)entry_slot[e] * state_stride;
    float acc = conv_b ? conv_b[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int src = i - (taps - 1 - j);
        const float v = src >= 0 ? proj[(size_t)(first + src) * proj_stride + x_off + c]
                                 : tail[(size_t)(taps - 1 + src) * CH + c];
        acc = fmaf(conv_w[(size_t)c * taps + j], v, acc);
    }
    u[(size_t)t * CH + c] = silu_f(acc);
}

__global__ void ssd_tail_kernel(const float* __restrict__ proj, int proj_stride, int x_off, int taps,
                                float* __restrict__ state, long long state_stride, const int* __restrict__ entry_q_start,
                                const int* __restrict__ entry_q_len, const int* __restrict__ entry_slot, int n_entries,
                                int CH) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_entries * CH) return;
    const int e = (int)(idx / CH), c = (int)(idx % CH);
    const int first = entry_q_start[e], n = entry_q_len[e];
    if (n <= 0) return;
    float* tail = state + (long long)entry_slot[e] * state_stride;
    float keep[MAX_TAPS];
#pragma unroll
    for (int r = 0; r < MAX_TAPS; ++r) {
        if (r < taps - 1) {
            const int src = n - (taps - 1) + r;
            keep[r] = src >= 0 ? proj[(size_t)(first + src) * proj_stride + x_off + c] : tail[(size_t)(n + r) * CH + c];
        }
    }
#pragma unroll
    for (int r = 0; r < MAX_TAPS; ++r)
        if (r < taps - 1) tail[(size_t)r * CH + c] = keep[r];
}

// mode 0: from the slot's state over all the request's tokens, outputs written, the slot's state updated.
// mode 1: chunk k of the request from S = 0, no outputs; end state and product of decays to chunk_state / chunk_decay.
// mode 2: chunk k from chunk_state[k], outputs written; the last chunk updates the slot.
// FULL: the state's rows are a multiple of 16, so a thread's 16 rows always exist and its B and C values are four aligned
// 16-byte loads; the arithmetic (and its order) is the same either way.
template <int MODE, bool FULL>
__global__ void ssd_scan_kernel(const float* __restrict__ u, int CH, const float* __restrict__ proj, int proj_stride,
                                int dt_off, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ skip, float* __restrict__ state, long long state_stride,
                                long long s_off, const int* __restrict__ entry_q_start, const int* __restrict__ entry_q_len,
                                const int* __restrict__ entry_slot, float* __restrict__ y, int heads, int groups, int N,
                                int P, int PT, int chunk_len, int max_chunks, float* __restrict__ chunk_state,
                                float* __restrict__ chunk_decay) {
    extern __shared__ float sm[];
    constexpr int mode = MODE;
    const int NJ = (N + NPT - 1) / NPT;
    float* xs = sm;                                  // [2][TCH][PT]
    float* Bs = xs + 2 * TCH * PT;                   // [2][TCH][N]
    float* Cs = Bs + 2 * TCH * N;                    // [2][TCH][N]
    float* dts = Cs + 2 * TCH * N;                   // [2][TCH]
    float* dec = dts + 2 * TCH;                      // [2][TCH]
    float* yp = dec + 2 * TCH;                       // [TCH][NJ][PT]
    const int e = blockIdx.x, h = blockIdx.y;
    const int pb = blockIdx.z % ((P + PT - 1) / PT), k = blockIdx.z / ((P + PT - 1) / PT);
    const int n_new = entry_q_len[e];
    int t0 = 0, t1 = n_new;
    if (mode != 0) {
        // a request is cut when its own portion is at least two chunks long, whatever else the step holds
        if (n_new >= 2 * chunk_len) {
            t0 = k * chunk_len;
            t1 = min(n_new, t0 + chunk_len);
        } else if (k > 0) {
            return;
        }
        if (t0 >= n_new) return;
        if (mode == 1 && t1 >= n_new) return;        // nobody reads the last chunk's end state from the scratch
    }
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int pl = tid % PT, j = tid / PT;
    const int p = pb * PT + pl;
    const bool live = p < P && j < NJ;
    const int first = entry_q_start[e];
    const int inner = heads * P;
    const int g = h / (heads / groups);
    float* S_slot = state + (long long)entry_slot[e] * state_stride + s_off + (size_t)h * N * P;
    const long long cs = (((long long)e * max_chunks + k) * heads + h) * (long long)N * P;
    const float rate = expf(a_log[h]), bias = dt_bias[h], dskip = skip[h];

    float S[NPT];
#pragma unroll
    for (int r = 0; r < NPT; ++r) {
        const int n = j * NPT + r;
        float v = 0.f;
        if (live && n < N) {
            if (mode == 0) v = S_slot[(size_t)n * P + p];
            else if (mode == 2) v = chunk_state[cs + (size_t)n * P + p];      // the chain left every chunk's start there
        }
        S[r] = v;
    }
    float total_decay = 1.f;

    // a stage: TCH tokens' x (this block's columns), B, C, step size and decay; filled by asynchronous copies
    // (no division in here: thread row j takes tokens j, j + rows, ...; warp w the B and C rows of tokens w, w + warps, ...)
    const int trows = nthr / PT, warp = tid >> 5, lane = tid & 31, nwarps = nthr >> 5;
    const bool wide = FULL && (inner & 3) == 0;      // rows of B and C start on 16-byte boundaries
    auto fill = [&](int c0, int buf) {
        const int nt = min(TCH, t1 - c0);
        float* xb = xs + buf * TCH * PT;
        float* Bb = Bs + buf * TCH * N;
        float* Cb = Cs + buf * TCH * N;
        if (j < trows) {
            for (int tt = j; tt < nt; tt += trows) {
                if (p < P) copy4_async(xb + tt * PT + pl, u + (size_t)(first + c0 + tt) * CH + (size_t)h * P + p);
                else xb[tt * PT + pl] = 0.f;
            }
        }
        for (int tt = warp; tt < nt; tt += nwarps) {
            const float* row = u + (size_t)(first + c0 + tt) * CH + inner + (size_t)g * N;
            if (wide) {
                for (int n = lane * 4; n < N; n += 128) {
                    copy16_async(Bb + tt * N + n, row + n);
                    copy16_async(Cb + tt * N + n, row + (size_t)groups * N + n);
                }
            } else {
                for (int n = lane; n < N; n += 32) {
                    copy4_async(Bb + tt * N + n, row + n);
                    copy4_async(Cb + tt * N + n, row + (size_t)groups * N + n);
                }
            }
        }
        if (tid < nt) {
            const float d = softplus_f(proj[(size_t)(first + c0 + tid) * proj_stride + dt_off + h] + bias);
            dts[buf * TCH + tid] = d;
            dec[buf * TCH + tid] = expf(-rate * d);
        }
    };
    fill(t0, 0);
    copies_commit();
    int buf = 0;
    for (int c0 = t0; c0 < t1; c0 += TCH, buf ^= 1) {
        const int nt = min(TCH, t1 - c0);
        if (c0 + TCH < t1) fill(c0 + TCH, buf ^ 1);  // (the other stage was let go of at the end of the pass before)
        copies_commit();
        copies_wait_all_but_one();
        __syncthreads();                             // this stage has landed, for every thread
        const float* xb = xs + buf * TCH * PT;
        for (int tt = 0; tt < nt; ++tt) {
            const float a = dec[buf * TCH + tt], dx = dts[buf * TCH + tt] * xb[tt * PT + pl];
            const float* Bt = Bs + (buf * TCH + tt) * N + j * NPT;
            const float* Ct = Cs + (buf * TCH + tt) * N + j * NPT;
            float acc = 0.f;
            if (j < NJ) {
                if (FULL) {
                    const float4* B4 = reinterpret_cast<const float4*>(Bt);
                    const float4* C4 = reinterpret_cast<const float4*>(Ct);
#pragma unroll
                    for (int q = 0; q < NPT / 4; ++q) {
                        const float4 b = B4[q];
                        S[4 * q] = fmaf(a, S[4 * q], b.x * dx);
                        S[4 * q + 1] = fmaf(a, S[4 * q + 1], b.y * dx);
                        S[4 * q + 2] = fmaf(a, S[4 * q + 2], b.z * dx);
                        S[4 * q + 3] = fmaf(a, S[4 * q + 3], b.w * dx);
                        if (mode != 1) {
                            const float4 c = C4[q];
                            acc = fmaf(S[4 * q], c.x, acc);
                            acc = fmaf(S[4 * q + 1], c.y, acc);
                            acc = fmaf(S[4 * q + 2], c.z, acc);
                            acc = fmaf(S[4 * q + 3], c.w, acc);
                        }
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < NPT; ++r) {
                        if (j * NPT + r < N) {
                            S[r] = fmaf(a, S[r], Bt[r] * dx);
                            if (mode != 1) acc = fmaf(S[r], Ct[r], acc);
                        }
                    }
                }
                if (mode != 1) yp[(tt * NJ + j) * PT + pl] = acc;
            }
            total_decay *= a;
        }
        if (mode != 1) {
            __syncthreads();
            if (j < trows && p < P) {
                for (int tt = j; tt < nt; tt += trows) {
                    float acc = 0.f;
                    for (int jj = 0; jj < NJ; ++jj) acc += yp[(tt * NJ + jj) * PT + pl];
                    y[(size_t)(first + c0 + tt) * inner + (size_t)h * P + p] = fmaf(dskip, xb[tt * PT + pl], acc);
                }
            }
        }
        __syncthreads();                             // this stage and the partial products may be overwritten
    }
    if (!live) return;
    if (mode == 1) {
#pragma unroll
        for (int r = 0; r < NPT; ++r)
            if (j * NPT + r < N) chunk_state[cs + (size_t)(j * NPT + r) * P + p] = S[r];
        if (tid == 0 && pb == 0) chunk_decay[((long long)e * max_chunks + k) * heads + h] = total_decay;
    } else if (t1 >= n_new) {
#pragma unroll
        for (int r = 0; r < NPT; ++r)
            if (j * NPT + r < N) S_slot[(size_t)(j * NPT + r) * P + p] = S[r];
    }
}

// chunk_state[k] (the end state of chunk k run from zero) becomes the state at the start of chunk k + 1, in place one
// slot later:  start[0] = the slot's state;  start[k + 1] = decay[k] * start[k] + end[k].  One thread per element of S.
__global__ void ssd_chain_kernel(const float* __restrict__ state, long long state_stride, long long s_off,
                                 const int* __restrict__ entry_q_len, const int* __restrict__ entry_slot,
                                 float* __restrict__ chunk_state, const float* __restrict__ chunk_decay, int heads,
                                 long long per_head, int chunk_len, int max_chunks) {
    const int e = blockIdx.y;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= heads * per_head) return;
    const int h = (int)(i / per_head);
    const int n_new = entry_q_len[e];
    const int n_chunks = n_new >= 2 * chunk_len ? (n_new + chunk_len - 1) / chunk_len : (n_new > 0 ? 1 : 0);
    float cur = state[(long long)entry_slot[e] * state_stride + s_off + i];
    constexpr int AHEAD = 8;                         // end states and decays of eight chunks are fetched together
    for (int k0 = 0; k0 + 1 < n_chunks; k0 += AHEAD) {
        float end[AHEAD], dec[AHEAD];
#pragma unroll
        for (int a = 0; a < AHEAD; ++a) {
            const int k = k0 + a;
            if (k + 1 < n_chunks) {
                end[a] = chunk_state[((long long)e * max_chunks + k) * heads * per_head + i];
                dec[a] = chunk_decay[((long long)e * max_chunks + k) * heads + h];
            }
        }
#pragma unroll
        for (int a = 0; a < AHEAD; ++a) {
            const int k = k0 + a;
            if (k + 1 < n_chunks) {
                chunk_state[((long long)e * max_chunks + k) * heads * per_head + i] = cur;      // chunk k starts from here
                cur = fmaf(dec[a], cur, end[a]);
            }
        }
    }
    if (n_chunks > 0) chunk_state[((long long)e * max_chunks + n_chunks - 1) * heads * per_head + i] = cur;
}

template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, int y_stride, const float* __restrict__ gate,
                                        int gate_stride, const float* __restrict__ weight, float eps, float scale,
                                        T* __restrict__ out, int out_stride, int n, int parts) {
    __shared__ float red[32];
    const int t = blockIdx.x, part = blockIdx.y;
    const int len = n / parts, c0 = part * len;
    const float* yr = y + (size_t)t * y_stride + c0;
    const float* gr = gate ? gate + (size_t)t * gate_stride + c0 : nullptr;
    float sq = 0.f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float v = gr ? yr[i] * silu_f(gr[i]) : yr[i];
        sq = fmaf(v, v, sq);
    }
    const float r = 1.0f / sqrtf(block_sum(sq, red) / (float)len + eps);
    T* o = out + (size_t)t * out_stride + c0;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float v = gr ? yr[i] * silu_f(gr[i]) : yr[i];
        o[i] = from_f32<T>(v * r * weight[c0 + i] * scale);
    }
}

}  // namespace

extern "C" {

int infero_ssd_state_floats(int heads, int N, int P, int groups, int taps) {
    return (taps - 1) * (heads * P + 2 * groups * N) + heads * N * P;
}

// u float32 [T, CH] receives silu(conv([x | B | C])); then the slot's tail moves on.
int infero_ssd_conv(const float* proj, int proj_stride, int x_off, const float* conv_w, const float* conv_b, int taps,
                    float* state, long long state_stride, const int* tok_entry, const int* entry_q_start,
                    const int* entry_q_len, const int* entry_slot, float* u, int n_tokens, int n_entries, int CH,
                    cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "ssd: %d taps outside 1..%d", taps, MAX_TAPS);
    const long long total = (long long)n_tokens * CH;
    ssd_conv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(proj, proj_stride, x_off, conv_w, conv_b, taps, state,
                                                                       state_stride, tok_entry, entry_q_start, entry_slot, u,
                                                                       n_tokens, CH);
    if (taps > 1) {
        const long long per = (long long)n_entries * CH;
        ssd_tail_kernel<<<(unsigned)((per + 255) / 256), 256, 0, stream>>>(proj, proj_stride, x_off, taps, state, state_stride,
                                                                         entry_q_start, entry_q_len, entry_slot, n_entries, CH);
    }
    return infero_check_launch("ssd_conv");
}

// Floats of scratch the chunked scan needs (0: the step runs unchunked).  A portion is cut into chunks when it is at
// least 2 * chunk_len long; how a request is cut depends on its own portion alone.
int infero_ssd_chunk_len() { return 128; }
long long infero_ssd_scan_scratch(int n_entries, int max_q_len, int heads, int N, int P) {
    const int L = infero_ssd_chunk_len();
    if (max_q_len < 2 * L) return 0;
    const long long chunks = (max_q_len + L - 1) / L;
    return (long long)n_entries * chunks * heads * ((long long)N * P + 1);
}

// y float32 [T, heads * P].  u as left by infero_ssd_conv; dt in proj at dt_off.
int infero_ssd_scan(const float* u, const float* proj, int proj_stride, int dt_off, const float* dt_bias,
                    const float* a_log, const float* skip, float* state, long long state_stride, int taps,
                    const int* entry_q_start, const int* entry_q_len, const int* entry_slot, float* y, int n_entries,
                    int max_q_len, int heads, int groups, int N, int P, float* scratch, int sm_count,
                    cudaStream_t stream) {
    if (n_entries == 0) return 0;
    INFERO_REQUIRE(groups >= 1 && heads % groups == 0, "ssd: %d heads do not split into %d groups", heads, groups);
    INFERO_REQUIRE(N >= 1 && N <= 16 * NPT, "ssd: a state of %d rows, at most %d", N, 16 * NPT);
    INFERO_REQUIRE(n_entries <= 65535 && heads <= 65535, "ssd: %d requests x %d heads are too many for one launch", n_entries, heads);
    const int CH = heads * P + 2 * groups * N;
    const long long s_off = (long long)(taps - 1) * CH;
    const int NJ = (N + NPT - 1) / NPT;
    const int L = infero_ssd_chunk_len();
    const int sms = sm_count > 0 ? sm_count : 148;
    // Columns of S per block: all of them up to 64, fewer (down to 8) while the grid would leave multiprocessors idle.
    // Blocks over the columns cost nothing extra, chunks cost a second pass: a step is cut into chunks only when
    // requests, heads and column blocks together do not fill the device.
    auto pick = [&](int chunks) {
        int pt = P < 64 ? P : 64;
        while (pt > 8 && pt % 2 == 0 && (long long)n_entries * heads * chunks * ((P + pt - 1) / pt) < 2ll * sms) pt /= 2;
        return pt;
    };
    int PT = pick(1);
    static const int chunk_rule = [] { const char* e = getenv("INFERO_SSD_CHUNKS"); return e ? atoi(e) : 1; }();
    // INFERO_SSD_CHUNKS: 1 (default) long portions always run by chunks; 2 only where the grid would not fill the device; 0 never
    const bool chunked = scratch != nullptr && max_q_len >= 2 * L && chunk_rule != 0 &&
                         (chunk_rule == 1 || (long long)n_entries * heads * ((P + PT - 1) / PT) < sms);
    const int max_chunks = chunked ? (max_q_len + L - 1) / L : 1;
    if (chunked) PT = pick(max_chunks);
    static const int max_threads = [] { const char* e = getenv("INFERO_SSD_THREADS"); return e ? atoi(e) : 256; }();
    // (256 threads a block measured best: three blocks' registers fit a multiprocessor; INFERO_SSD_THREADS changes it)
    while (PT * NJ > max_threads && PT > 1) PT = (PT + 1) / 2;
    const int pbs = (P + PT - 1) / PT;
    const int threads = ((PT * NJ + 31) / 32) * 32;
    const size_t smem = (size_t)TCH * (2 * (PT + 2 * N + 2) + NJ * PT) * sizeof(float);
    INFERO_REQUIRE(smem <= 200 * 1024, "ssd: state %d x %d needs %zu bytes of shared memory", N, P, smem);
    const bool full = N % NPT == 0;
    auto k0 = full ? ssd_scan_kernel<0, true> : ssd_scan_kernel<0, false>;
    auto k1 = full ? ssd_scan_kernel<1, true> : ssd_scan_kernel<1, false>;
    auto k2 = full ? ssd_scan_kernel<2, true> : ssd_scan_kernel<2, false>;
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    float* chunk_state = scratch;
    float* chunk_decay = scratch ? scratch + (long long)n_entries * max_chunks * heads * N * P : nullptr;
    if (!chunked) {
        k0<<<dim3(n_entries, heads, pbs), threads, smem, stream>>>(
            u, CH, proj, proj_stride, dt_off, dt_bias, a_log, skip, state, state_stride, s_off, entry_q_start, entry_q_len,
            entry_slot, y, heads, groups, N, P, PT, 0, 1, nullptr, nullptr);
        return infero_check_launch("ssd_scan");
    }
    INFERO_REQUIRE((long long)pbs * max_chunks <= 65535, "ssd: a portion of %d tokens is too long for one launch", max_q_len);
    const dim3 grid(n_entries, heads, pbs * max_chunks);
    k1<<<grid, threads, smem, stream>>>(u, CH, proj, proj_stride, dt_off, dt_bias, a_log, skip, state, state_stride,
                                                       s_off, entry_q_start, entry_q_len, entry_slot, y, heads, groups, N, P, PT,
                                                       L, max_chunks, chunk_state, chunk_decay);
    const long long per_head = (long long)N * P;
    ssd_chain_kernel<<<dim3((unsigned)((heads * per_head + 255) / 256), n_entries), 256, 0, stream>>>(
        state, state_stride, s_off, entry_q_len, entry_slot, chunk_state, chunk_decay, heads, per_head, L, max_chunks);
    k2<<<grid, threads, smem, stream>>>(u, CH, proj, proj_stride, dt_off, dt_bias, a_log, skip, state, state_stride,
                                                       s_off, entry_q_start, entry_q_len, entry_slot, y, heads, groups, N, P, PT,
                                                       L, max_chunks, chunk_state, chunk_decay);
    return infero_check_launch("ssd_scan_chunked");
}

// out[t, c] = v / sqrt(mean over c's part of v^2 + eps) * weight[c] * scale with v = y[t, c] * silu(gate[t, c]) (v = y
// without a gate); the n columns form `parts` equal parts.  y, gate float32 with free row strides; out of `dtype`.
int infero_gated_group_norm(const float* y, int y_stride, const float* gate, int gate_stride, const float* weight, float eps,
                            float scale, void* out, int out_stride, int dtype, int n_tokens, int n, int parts,
                            cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(parts >= 1 && n % parts == 0 && parts <= 65535, "group norm: %d columns do not split into %d parts", n, parts);
    const int len = n / parts;
    const int threads = len >= 512 ? 256 : len >= 128 ? 128 : 64;
    const dim3 grid(n_tokens, parts);
    if (dtype == INFERO_F32)
        gated_group_norm_kernel<float><<<grid, threads, 0, stream>>>(y, y_stride, gate, gate_stride, weight, eps, scale,
                                                                    (float*)out, out_stride, n, parts);
    else
        gated_group_norm_kernel<bf16><<<grid, threads, 0, stream>>>(y, y_stride, gate, gate_stride, weight, eps, scale,
                                                                   (bf16*)out, out_stride, n, parts);
    return infero_check_launch("gated_group_norm");
}

}  // extern "C"

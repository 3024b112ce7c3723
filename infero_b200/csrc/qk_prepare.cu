// Between a layer's input product and attention over the paged cache, for mixers whose queries and keys are normed:
// per token, from the 32-bit product row (biases already added),
//
//   norm 0: none
//   norm 1: RMS norm over the whole query projection (all heads at once) with a weight per coordinate, and likewise
//           over the whole key projection, before the rotation
//   norm 2: every head of q and k divided by its root mean square (no weight), after the rotation
//   norm 3: an RMS norm over every head of q and of k with a weight of D numbers shared by the heads (one for q, one
//           for k), before the rotation
//
//   rotation: the first `rot` coordinates of every head, coordinate i with i + rot/2, by position * freq[i]; the angle
//   is formed in 64-bit from a 64-bit table made on the host (any scaling of the frequencies is the host's) and brought
//   into [-pi, pi] before sincosf; cos and sin are multiplied by `amp`.
//
//   values: a projection of their own (v_off >= 0), or the keys as projected, before norm and rotation (v_off < 0).
//
// The query goes to q_out in the step's element type, keys and values to the token's page (write_cache; a layer that
// reads another layer's cache has no key or value columns at all).  One block per token; the row is staged in shared
// memory, the sines of a token are worked out once for all heads.  Everything is 32-bit up to the final store.
//
// head_gate: out[t, h * V + v] = a[t, h * V + v] * sigmoid(g[t, h]) * scale, the sigmoid gate per head that such a mixer
// may put on its result.
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS)
qk_prepare_kernel(const float* __restrict__ proj, int proj_stride, int q_off, int k_off, int v_off, int norm_mode,
                  const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_w_dtype, float eps,
                  const double* __restrict__ freq, int rot, float amp, const int* __restrict__ positions,
                  const int* __restrict__ tok_entry, const int* __restrict__ block_table, int max_blocks, int page_size,
                  T* __restrict__ q_out, int q_stride, T* __restrict__ k_cache, T* __restrict__ v_cache, int write_cache,
                  int H, int G, int D, int V) {
    extern __shared__ float smem[];
    __shared__ float red[32];
    const int half = rot / 2;
    float* buf = smem;                               // [(H + Gk) * D]: q heads, then k heads
    const int Gk = write_cache ? G : 0;
    float* cs = buf + (size_t)(H + Gk) * D;          // [half] cos, [half] sin
    float* sn = cs + half;
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* row = proj + (size_t)t * proj_stride;
    const int pos = positions[t];
    const int nq = H * D, nk = Gk * D;

    for (int i = tid; i < nq; i += THREADS) buf[i] = row[q_off + i];
    for (int i = tid; i < nk; i += THREADS) buf[nq + i] = row[k_off + i];
    for (int i = tid; i < half; i += THREADS) {
        const double two_pi = 6.283185307179586476925286766559;
        double ang = (double)pos * freq[i];
        ang -= two_pi * rint(ang / two_pi);
        float s, c;
        sincosf((float)ang, &s, &c);
        cs[i] = c * amp, sn[i] = s * amp;
    }
    long long page_row = -1;                          // row of this token in the cache arrays, per kv head 0
    if (write_cache) {
        const int page = block_table[(size_t)tok_entry[t] * max_blocks + pos / page_size];
        page_row = (long long)page * G * page_size + (pos % page_size);
    }
    __syncthreads();
    if (write_cache) {
        // values: their own projection, or the keys as they were projected
        if (v_off >= 0) {
            for (int i = tid; i < G * V; i += THREADS) {
                const int g = i / V, c = i % V;
                v_cache[(page_row + (long long)g * page_size) * V + c] = from_f32<T>(row[v_off + i]);
            }
        } else {
            for (int i = tid; i < nk; i += THREADS) {
                const int g = i / D, c = i % D;
                v_cache[(page_row + (long long)g * page_size) * V + c] = from_f32<T>(buf[nq + i]);
            }
        }
    }
    if (norm_mode == 1) {
        float sq = 0.f, sk = 0.f;
        for (int i = tid; i < nq; i += THREADS) sq = fmaf(buf[i], buf[i], sq);
        for (int i = tid; i < nk; i += THREADS) sk = fmaf(buf[nq + i], buf[nq + i], sk);
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        const float rq = 1.0f / sqrtf(sq / (float)nq + eps);
        const float rk = nk ? 1.0f / sqrtf(sk / (float)nk + eps) : 0.f;
        __syncthreads();
        for (int i = tid; i < nq; i += THREADS) buf[i] = buf[i] * rq * load_any(q_norm_w, norm_w_dtype, i);
        for (int i = tid; i < nk; i += THREADS) buf[nq + i] = buf[nq + i] * rk * load_any(k_norm_w, norm_w_dtype, i);
    }
    if (norm_mode == 3) {
        const int warp = tid >> 5, lane = tid & 31;
        for (int head = warp; head < H + Gk; head += THREADS / 32) {
            float* hp = buf + (size_t)head * D;
            const void* w = head < H ? q_norm_w : k_norm_w;
            float s = 0.f;
            for (int i = lane; i < D; i += 32) s = fmaf(hp[i], hp[i], s);
            s = warp_sum(s);
            const float r = 1.0f / sqrtf(s / (float)D + eps);
            for (int i = lane; i < D; i += 32) hp[i] = hp[i] * r * load_any(w, norm_w_dtype, i);
        }
    }
    __syncthreads();
    // rotation: a thread owns a pair, so nothing is read after it was rewritten
    for (int e = tid; e < (H + Gk) * half; e += THREADS) {
        const int head = e / half, i = e % half;
        float* hp = buf + (size_t)head * D;
        const float a = hp[i], b = hp[i + half];
        hp[i] = a * cs[i] - b * sn[i];
        hp[i + half] = b * cs[i] + a * sn[i];
    }
    __syncthreads();
    if (norm_mode == 2) {
        const int warp = tid >> 5, lane = tid & 31;
        for (int head = warp; head < H + Gk; head += THREADS / 32) {
            float* hp = buf + (size_t)head * D;
            float s = 0.f;
            for (int i = lane; i < D; i += 32) s = fmaf(hp[i], hp[i], s);
            s = warp_sum(s);
            const float r = 1.0f / sqrtf(s / (float)D + eps);
            for (int i = lane; i < D; i += 32) hp[i] *= r;
        }
        __syncthreads();
    }
    T* qo = q_out + (size_t)t * q_stride;
    for (int i = tid; i < nq; i += THREADS) qo[i] = from_f32<T>(buf[i]);
    for (int i = tid; i < nk; i += THREADS) {
        const int g = i / D, c = i % D;
        k_cache[(page_row + (long long)g * page_size) * D + c] = from_f32<T>(buf[nq + i]);
    }
}

template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ a, int a_stride, const float* __restrict__ gate, int gate_stride,
                                 T* __restrict__ out, int out_stride, int n_tokens, int H, int V, float scale) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * H * V) return;
    const int t = (int)(i / (H * V)), c = (int)(i % (H * V)), h = c / V;
    float v = to_f32(a[(size_t)t * a_stride + c]) * scale;
    if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + h]));
    out[(size_t)t * out_stride + c] = from_f32<T>(v);
}

// Eight neighbouring columns a thread (they lie in one head when V is a multiple of 8): 16-byte loads and stores.
__global__ void head_gate_vec_kernel(const bf16* __restrict__ a, int a_stride, const float* __restrict__ gate, int gate_stride,
                                     bf16* __restrict__ out, int out_stride, int n_tokens, int H, int V, float scale) {
    const int per_row = H * V / 8;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * per_row) return;
    const int t = (int)(i / per_row), c = (int)(i % per_row) * 8, h = c / V;
    float f = scale;
    if (gate) f *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + h]));
    const uint4 v = *reinterpret_cast<const uint4*>(a + (size_t)t * a_stride + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
        const __nv_bfloat162 p = __floats2bfloat162_rn(lo * f, hi * f);
        r[j] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * out_stride + c) = make_uint4(r[0], r[1], r[2], r[3]);
}

}  // namespace

extern "C" {

int infero_qk_prepare(const float* proj, int proj_stride, int q_off, int k_off, int v_off, int norm_mode,
                      const void* q_norm_w, const void* k_norm_w, int norm_w_dtype, float eps, const double* freq,
                      int rot, float amp, const int* positions, const int* tok_entry, const int* block_table,
                      int max_blocks, int page_size, void* q_out, int q_stride, void* k_cache, void* v_cache, int dtype,
                      int write_cache, int n_tokens, int H, int G, int D, int V, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    INFERO_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= D, "qk_prepare: %d rotated coordinates of %d", rot, D);
    INFERO_REQUIRE(norm_mode >= 0 && norm_mode <= 3, "qk_prepare: norm mode %d", norm_mode);
    INFERO_REQUIRE((norm_mode != 1 && norm_mode != 3) || (q_norm_w && (!write_cache || k_norm_w)), "qk_prepare: norm weights missing");
    INFERO_REQUIRE(v_off >= 0 || V == D || !write_cache, "qk_prepare: values taken from keys need equal widths (%d, %d)", V, D);
    const size_t smem = ((size_t)(H + (write_cache ? G : 0)) * D + rot) * sizeof(float);
    INFERO_REQUIRE(smem <= 200 * 1024, "qk_prepare: %d heads of %d do not fit in shared memory", H + G, D);
#define LAUNCH(T)                                                                                                        \
    do {                                                                                                                 \
        auto k = qk_prepare_kernel<T>;                                                                                   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        k<<<n_tokens, THREADS, smem, stream>>>(proj, proj_stride, q_off, k_off, v_off, norm_mode, q_norm_w, k_norm_w,    \
                                               norm_w_dtype, eps, freq, rot, amp, positions, tok_entry, block_table,      \
                                               max_blocks, page_size, (T*)q_out, q_stride, (T*)k_cache, (T*)v_cache,      \
                                               write_cache, H, G, D, V);                                                  \
    } while (0)
    if (dtype == INFERO_F32) LAUNCH(float);
    else LAUNCH(bf16);
#undef LAUNCH
    return infero_check_launch("qk_prepare");
}

int infero_head_gate(const void* a, int a_stride, const float* gate, int gate_stride, void* out, int out_stride, int dtype,
                     int n_tokens, int H, int V, float scale, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    const long long total = (long long)n_tokens * H * V;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (dtype != INFERO_F32 && V % 8 == 0 && a_stride % 8 == 0 && out_stride % 8 == 0 && al16(a) && al16(out)) {
        head_gate_vec_kernel<<<(unsigned)((total / 8 + 255) / 256), 256, 0, stream>>>((const bf16*)a, a_stride, gate, gate_stride,
                                                                                     (bf16*)out, out_stride, n_tokens, H, V, scale);
        return infero_check_launch("head_gate");
    }
    if (dtype == INFERO_F32)
        head_gate_kernel<float><<<blocks, 256, 0, stream>>>((const float*)a, a_stride, gate, gate_stride, (float*)out,
                                                             out_stride, n_tokens, H, V, scale);
    else
        head_gate_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)a, a_stride, gate, gate_stride, (bf16*)out,
                                                            out_stride, n_tokens, H, V, scale);
    return infero_check_launch("head_gate");
}

}  // extern "C"

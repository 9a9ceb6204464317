// Grouped-query attention whose keys and values differ in width, with a window that keeps the first positions of a
// request and a learned sink per head in the softmax denominator: the step between the projections and the cache
// (norm over the whole projection, partial rotation, cache write) and the plain attention kernel (one warp per
// (token, query head), any sizes, both types: the 32-bit path, the fallback and the twin of the tensor-core kernel).
//
// A cache page holds the keys of its tokens, [nkv][page_size][dk], and behind them the values, [nkv][page_size][dv].
// A token's result depends only on its own query and the keys of its request, never on what else is in the launch.
#include "common.cuh"
#include "kernel_args.h"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

// ----------------------------------------------------------------------------- norm, rotation, cache write
// One value of a projection row after the norm (x * rinv * gain) and the rotation of its head's first `dims`
// coordinates in rotate-half pairs (i, i + dims/2) by position * inv_freq[i], cosine and sine times `amp`.
// `interleaved`: the pairs are (2i, 2i + 1) instead.
template <typename T>
__device__ __forceinline__ float finished_value(const T* __restrict__ row, const float* __restrict__ gain, float rinv, int head, int d, int dk,
                                                const float* __restrict__ inv_freq, int dims, float amp, int position, int interleaved) {
    const int base = head * dk;
    auto normed = [&](int j) -> float {
        const float v = to_f32(row[base + j]);
        return gain ? (v * rinv) * gain[base + j] : v;
    };
    if (!inv_freq || d >= dims) return normed(d);
    const int half = dims >> 1, i = interleaved ? d >> 1 : (d < half ? d : d - half);
    float s, c;
    sincosf((float)position * inv_freq[i], &s, &c);
    s *= amp;
    c *= amp;
    const float u = normed(interleaved ? 2 * i : i), w = normed(interleaved ? 2 * i + 1 : i + half);
    const bool first = interleaved ? !(d & 1) : d < half;
    return first ? u * c - w * s : w * c + u * s;
}

// I: the type of the projections (that of everything else, or 32-bit where they come from a convolution); T: the type of the
// finished queries and of the cache.
template <typename I, typename T>
__global__ void window_post_kernel(LlmeWindowPostArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x, dk = a.dk, dv = a.dv, ps = a.page_size;
    const int pos = a.positions[t];
    const int qn = a.nh * dk, kn = a.nkv * dk, vn = a.nkv * dv;
    const I* q = (const I*)a.q_in + (size_t)t * a.q_stride;
    float rq = 1.0f, rk = 1.0f;
    if (a.q_gain) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < qn; j += blockDim.x) {
            const float v = to_f32(q[j]);
            ss += v * v;
        }
        rq = 1.0f / sqrtf(block_sum(ss, scratch) / (float)qn + a.eps);
    }
    T* qo = (T*)a.q_out + (size_t)t * qn;
    for (int j = threadIdx.x; j < qn; j += blockDim.x)
        qo[j] = from_f32<T>(finished_value(q, a.q_gain, rq, j / dk, j % dk, dk, a.inv_freq, a.rot_dims, a.amplitude, pos, a.interleaved));
    const int slot = (a.cache && a.slot_mapping) ? a.slot_mapping[t] : -1;
    if (!a.k_in || slot < 0) return;                    // uniform over the block
    const I* k = (const I*)a.k_in + (size_t)t * a.k_stride;
    const I* v = (const I*)a.v_in + (size_t)t * a.v_stride;
    if (a.k_gain) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < kn; j += blockDim.x) {
            const float x = to_f32(k[j]);
            ss += x * x;
        }
        rk = 1.0f / sqrtf(block_sum(ss, scratch) / (float)kn + a.eps);
    }
    const int page = slot / ps, off = slot - page * ps;
    T* kpage = (T*)a.cache + (size_t)page * ((size_t)a.nkv * ps * (dk + dv));
    T* vpage = kpage + (size_t)a.nkv * ps * dk;
    for (int j = threadIdx.x; j < kn; j += blockDim.x) {
        const int g = j / dk, d = j - g * dk;
        kpage[((size_t)g * ps + off) * dk + d] = from_f32<T>(finished_value(k, a.k_gain, rk, g, d, dk, a.inv_freq, a.rot_dims, a.amplitude, pos, a.interleaved));
    }
    for (int j = threadIdx.x; j < vn; j += blockDim.x) {
        const int g = j / dv, d = j - g * dv;
        vpage[((size_t)g * ps + off) * dv + d] = from_f32<T>(to_f32(v[j]));
    }
}

// The same step for designs that norm every head by itself (gains of one head's size, shared by the heads) and whose
// projections have biases: one warp per (token, head); the biased head is read twice (sum of squares, then the values).
// The value may be the key's own projection (v_in = k_in): it is stored as projected, with its bias, before the norm.
template <typename T>
__device__ __forceinline__ void finish_head(const T* __restrict__ in, const float* __restrict__ bias, const float* __restrict__ gain, float eps, int dk,
                                            const float* __restrict__ inv_freq, int dims, float amp, int position, T* __restrict__ out, int lane,
                                            int interleaved) {
    auto raw = [&](int j) -> float {
        const float v = to_f32(in[j]);
        return bias ? to_f32(from_f32<T>(v + bias[j])) : v;      // a projection's output has the type of the products
    };
    float rinv = 1.0f;
    if (gain) {
        float ss = 0.0f;
        for (int j = lane; j < dk; j += 32) {
            const float v = raw(j);
            ss += v * v;
        }
        rinv = 1.0f / sqrtf(warp_sum(ss) / (float)dk + eps);
    }
    auto normed = [&](int j) -> float { return gain ? (raw(j) * rinv) * gain[j] : raw(j); };
    const int half = dims >> 1;
    for (int d = lane; d < dk; d += 32) {
        float v;
        if (!inv_freq || d >= dims) v = normed(d);
        else {
            const int i = interleaved ? d >> 1 : (d < half ? d : d - half);
            float s, c;
            sincosf((float)position * inv_freq[i], &s, &c);
            s *= amp;
            c *= amp;
            const float u = normed(interleaved ? 2 * i : i), w = normed(interleaved ? 2 * i + 1 : i + half);
            v = (interleaved ? !(d & 1) : d < half) ? u * c - w * s : w * c + u * s;
        }
        out[d] = from_f32<T>(v);
    }
}

template <typename T>
__global__ void window_post_heads_kernel(LlmeWindowPostArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * warps + (threadIdx.x >> 5);       // (token, head of q | head of k | head of v)
    const bool stores = a.k_in != nullptr;
    const int per_token = a.nh + (stores ? 2 * a.nkv : 0);
    if (item >= a.tokens * per_token) return;
    const int t = item / per_token, hh = item - t * per_token;
    const int dk = a.dk, dv = a.dv, ps = a.page_size, pos = a.positions[t];
    if (hh < a.nh) {
        finish_head((const T*)a.q_in + (size_t)t * a.q_stride + hh * dk, a.q_bias ? a.q_bias + hh * dk : nullptr, a.q_gain, a.eps, dk,
                    a.inv_freq, a.rot_dims, a.amplitude, pos, (T*)a.q_out + ((size_t)t * a.nh + hh) * dk, lane, a.interleaved);
        return;
    }
    const int slot = a.slot_mapping[t];
    if (slot < 0) return;
    const int page = slot / ps, off = slot - page * ps;
    T* kpage = (T*)a.cache + (size_t)page * ((size_t)a.nkv * ps * (dk + dv));
    if (hh < a.nh + a.nkv) {
        const int g = hh - a.nh;
        finish_head((const T*)a.k_in + (size_t)t * a.k_stride + g * dk, a.k_bias ? a.k_bias + g * dk : nullptr, a.k_gain, a.eps, dk,
                    a.inv_freq, a.rot_dims, a.amplitude, pos, kpage + ((size_t)g * ps + off) * dk, lane, a.interleaved);
        return;
    }
    const int g = hh - a.nh - a.nkv;
    const T* v = (const T*)a.v_in + (size_t)t * a.v_stride + g * dv;
    T* vo = kpage + (size_t)a.nkv * ps * dk + ((size_t)g * ps + off) * dv;
    for (int d = lane; d < dv; d += 32) vo[d] = a.v_bias ? from_f32<T>(to_f32(v[d]) + a.v_bias[g * dv + d]) : v[d];
}

LLME_API int llme_window_post(const LlmeWindowPostArgs* args, int dtype, cudaStream_t stream) {
    const LlmeWindowPostArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (!a.q_in || !a.q_out || !a.positions) LLME_REFUSE("window_post: null pointer");
    if ((a.k_in == nullptr) != (a.v_in == nullptr)) LLME_REFUSE("window_post: keys and values are stored together");
    if (a.k_in && (!a.cache || !a.slot_mapping || a.page_size <= 0)) LLME_REFUSE("window_post: keys without a cache to store them in");
    if (a.nh <= 0 || a.nkv <= 0 || a.dk <= 0 || a.dv <= 0) LLME_REFUSE("window_post: non-positive size");
    if (a.inv_freq && (a.rot_dims <= 0 || a.rot_dims % 2 || a.rot_dims > a.dk))
        LLME_REFUSE("window_post: %d rotated coordinates of %d need an even count", a.rot_dims, a.dk);
    if ((a.q_gain || a.k_gain) && !(a.eps > 0.0f)) LLME_REFUSE("window_post: eps must be positive");
    const bool wide_in = a.in_f32 && dtype != LLME_F32;     // 32-bit projections, everything else in the type of the products
    if (a.head_norm || a.q_bias || a.k_bias || a.v_bias) {
        if (wide_in) LLME_REFUSE("window_post: 32-bit projections come without biases and without the norm per head");
        if (!a.head_norm && (a.q_gain || a.k_gain)) LLME_REFUSE("window_post: biases come with the norm per head or with no norm");
        const long long items = (long long)a.tokens * (a.nh + (a.k_in ? 2 * a.nkv : 0));
        const int wpb = 4;
        if (dtype == LLME_F32) llme_launch(window_post_heads_kernel<float>, dim3((unsigned)((items + wpb - 1) / wpb)), dim3(wpb * 32), 0, stream, a);
        else if (dtype == LLME_BF16) llme_launch(window_post_heads_kernel<__nv_bfloat16>, dim3((unsigned)((items + wpb - 1) / wpb)), dim3(wpb * 32), 0, stream, a);
        else LLME_REFUSE("window_post: unsupported dtype %d", dtype);
        LLME_LAUNCH_STATUS();
    }
    const int qn = a.nh * a.dk;
    const int threads = qn >= 2048 ? 512 : (qn >= 512 ? 256 : 128);
    if (dtype == LLME_F32) llme_launch(window_post_kernel<float, float>, dim3(a.tokens), dim3(threads), 0, stream, a);
    else if (dtype == LLME_BF16 && wide_in) llme_launch(window_post_kernel<float, __nv_bfloat16>, dim3(a.tokens), dim3(threads), 0, stream, a);
    else if (dtype == LLME_BF16) llme_launch(window_post_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(a.tokens), dim3(threads), 0, stream, a);
    else LLME_REFUSE("window_post: unsupported dtype %d", dtype);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- plain attention
template <typename T, int KR, int VR>
__global__ void window_attention_plain_kernel(LlmeWindowAttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int h = blockIdx.y;
    if (t >= a.tokens) return;
    const int dk = a.dk, dv = a.dv, ps = a.page_size;
    const int kvh = h / (a.nh / a.nkv);
    const int p = a.positions[t];
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;
    const int first = a.keep_first < lo ? a.keep_first : lo;       // keys 0 .. first-1 are seen beside the window
    const int* bt = a.block_tables + (size_t)a.token_request[t] * a.max_blocks;
    const size_t page_elems = (size_t)a.nkv * ps * (dk + dv);

    float q[KR], acc[VR];
    const T* qp = (const T*)a.q + ((size_t)t * a.nh + h) * dk;
#pragma unroll
    for (int i = 0; i < KR; ++i) {
        const int d = lane + 32 * i;
        q[i] = d < dk ? to_f32(qp[d]) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < VR; ++i) acc[i] = 0.0f;
    // the sink is one more term of the denominator: a score that is not scaled and has no value
    float m = a.sink ? a.sink[h] : -INFINITY, l = a.sink ? 1.0f : 0.0f;
    for (int jj = 0; jj < first + (p - lo + 1); ++jj) {
        const int j = jj < first ? jj : lo + (jj - first);
        const int page = bt[j / ps];
        const int off = j - (j / ps) * ps;
        const T* kp = (const T*)a.cache + (size_t)page * page_elems + ((size_t)kvh * ps + off) * dk;
        const T* vp = (const T*)a.cache + (size_t)page * page_elems + (size_t)a.nkv * ps * dk + ((size_t)kvh * ps + off) * dv;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < KR; ++i) {
            const int d = lane + 32 * i;
            if (d < dk) s += q[i] * to_f32(kp[d]);
        }
        s = warp_sum(s) * a.scale;
        if (a.softcap > 0.0f) s = a.softcap * tanhf(s / a.softcap);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);       // exp(-inf) = 0 on the first key
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < VR; ++i) {
            const int d = lane + 32 * i;
            if (d < dv) acc[i] = acc[i] * corr + e * to_f32(vp[d]);
        }
        m = m_new;
    }
    T* op = (T*)a.out + ((size_t)t * a.nh + h) * dv;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < VR; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) op[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T, int KR>
static int launch_plain_v(const LlmeWindowAttnArgs& a, cudaStream_t s) {
    const int wpb = 4;
    dim3 grid((a.tokens + wpb - 1) / wpb, a.nh);
    const int regs = (a.dv + 31) / 32;
    if (regs <= 1) llme_launch(window_attention_plain_kernel<T, KR, 1>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 2) llme_launch(window_attention_plain_kernel<T, KR, 2>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 4) llme_launch(window_attention_plain_kernel<T, KR, 4>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 8) llme_launch(window_attention_plain_kernel<T, KR, 8>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else if (regs <= 16) llme_launch(window_attention_plain_kernel<T, KR, 16>, dim3(grid), dim3(wpb * 32), 0, s, a);
    else LLME_REFUSE("window attention: a value size of %d is larger than 512", a.dv);
    LLME_LAUNCH_STATUS();
}

template <typename T>
static int launch_plain(const LlmeWindowAttnArgs& a, cudaStream_t s) {
    const int regs = (a.dk + 31) / 32;
    if (regs <= 1) return launch_plain_v<T, 1>(a, s);
    if (regs <= 2) return launch_plain_v<T, 2>(a, s);
    if (regs <= 4) return launch_plain_v<T, 4>(a, s);
    if (regs <= 8) return launch_plain_v<T, 8>(a, s);
    if (regs <= 16) return launch_plain_v<T, 16>(a, s);
    LLME_REFUSE("window attention: a query/key size of %d is larger than 512", a.dk);
}

LLME_API int llme_window_attention_plain(const LlmeWindowAttnArgs* args, int dtype, cudaStream_t stream) {
    const LlmeWindowAttnArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (!a.q || !a.cache || !a.out || !a.positions || !a.token_request || !a.block_tables) LLME_REFUSE("window attention: null pointer");
    if (a.nh <= 0 || a.nkv <= 0 || a.nh % a.nkv) LLME_REFUSE("window attention: %d query heads are not a multiple of %d key/value heads", a.nh, a.nkv);
    if (a.dk <= 0 || a.dv <= 0 || a.page_size <= 0 || a.max_blocks <= 0 || a.window < 0 || a.keep_first < 0) LLME_REFUSE("window attention: bad size");
    if (a.nh > 65535) LLME_REFUSE("window attention: more than 65535 query heads");
    if (dtype == LLME_F32) return launch_plain<float>(a, stream);
    if (dtype == LLME_BF16) return launch_plain<__nv_bfloat16>(a, stream);
    LLME_REFUSE("window attention: unsupported dtype %d", dtype);
}

// Layers that carry a state of fixed size per request instead of a cache that grows: a short causal convolution per
// channel, the rotation of queries and keys into 32-bit, a linear recurrence with a decaying matrix state per head
// (linear attention with a fixed decay per head; a selective state space whose decay and step come with every token), and
// the grouped RMS norm with a silu gate that follows such a recurrence.  Everything that enters the recurrence is 32-bit,
// and so is the state; a request's tokens are taken in their order, so what a token gets does not depend on how its
// prompt was cut into steps or on what else the step holds.
#include "common.cuh"
#include "kernel_args.h"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
    return dtype == LLME_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__device__ __forceinline__ float silu32(float z) { return z / (1.0f + expf(-z)); }

// softplus(z) = max(z, 0) + log(1 + exp(-|z|)), no clamp
__device__ __forceinline__ float softplus32(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// The batch row of token t: the last r with cu[r] <= t.
__device__ __forceinline__ int row_of_token(const int* __restrict__ cu, int requests, int t) {
    int lo = 0, hi = requests;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// ----------------------------------------------------------------------------- short causal convolution
constexpr int MAX_TAPS = 16;

__global__ void short_conv_kernel(LlmeShortConvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, K = a.taps;
    const int r = row_of_token(a.cu_q_lens, a.requests, t);
    const int i = t - a.cu_q_lens[r];                       // place of the token in its request's portion
    const float* st = a.state + (size_t)a.state_slots[r] * a.state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.channels; c += gridDim.y * blockDim.x) {
        float y = a.bias ? a.bias[c] : 0.0f;
        for (int j = K - 1; j >= 0; --j) {                   // the oldest input first
            const int src = i - j;
            const float x = src >= 0 ? load_as_f32(a.x, a.x_dtype, (size_t)(t - j) * a.ldx + c)
                                     : st[(size_t)(K - 1 + src) * a.channels + c];
            y = fmaf(a.w[(size_t)c * K + (K - 1 - j)], x, y);
        }
        a.out[(size_t)t * a.ldo + c] = a.act == 1 ? silu32(y) : y;
    }
}

__global__ void short_conv_state_kernel(LlmeShortConvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, K = a.taps;
    const int first = a.cu_q_lens[r], n = a.cu_q_lens[r + 1] - first;
    float* st = a.state + (size_t)a.state_slots[r] * a.state_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.channels; c += gridDim.y * blockDim.x) {
        float old[MAX_TAPS];
#pragma unroll
        for (int m = 0; m < MAX_TAPS; ++m) old[m] = m < K - 1 ? st[(size_t)m * a.channels + c] : 0.0f;
#pragma unroll
        for (int m = 0; m < MAX_TAPS; ++m) {
            if (m >= K - 1) break;
            const int src = n - (K - 1) + m;                 // place in the portion of what slot m holds afterwards
            float v = 0.0f;
            if (src >= 0) v = load_as_f32(a.x, a.x_dtype, (size_t)(first + src) * a.ldx + c);
            else {
#pragma unroll
                for (int o = 0; o < MAX_TAPS; ++o) if (o == K - 1 + src) v = old[o];
            }
            st[(size_t)m * a.channels + c] = v;
        }
    }
}

LLME_API int llme_short_conv(const LlmeShortConvArgs* args, int update, cudaStream_t stream) {
    const LlmeShortConvArgs& a = *args;
    if (a.tokens <= 0 || a.requests <= 0 || a.channels <= 0) return 0;
    if (!a.x || !a.w || !a.state || !a.out || !a.cu_q_lens || !a.state_slots) LLME_REFUSE("short_conv: null pointer");
    if (a.taps < 1 || a.taps > MAX_TAPS) LLME_REFUSE("short_conv: %d taps, this build takes 1 to %d", a.taps, MAX_TAPS);
    if (a.x_dtype != LLME_F32 && a.x_dtype != LLME_BF16) LLME_REFUSE("short_conv: unsupported dtype %d", a.x_dtype);
    const int threads = 128;
    int pieces = (a.channels + threads - 1) / threads;
    if (update) {
        if (a.taps > 1) llme_launch(short_conv_state_kernel, dim3(a.requests, pieces), dim3(threads), 0, stream, a);
    } else {
        const int wanted = (592 + a.tokens - 1) / a.tokens;
        if (pieces > wanted) pieces = wanted;
        llme_launch(short_conv_kernel, dim3(a.tokens, pieces < 1 ? 1 : pieces), dim3(threads), 0, stream, a);
    }
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- rotation into 32-bit
__global__ void rotate_kernel(LlmeRotateArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, pos = a.positions[t], half = a.rot_dims >> 1;
    for (int which = 0; which < 2; ++which) {
        if (!a.x[which]) continue;
        const int total = a.heads[which] * a.dim;
        const size_t in = (size_t)t * a.ldx[which];
        float* o = a.out[which] + (size_t)t * a.ldo[which];
        for (int e = threadIdx.x; e < total; e += blockDim.x) {
            const int h = e / a.dim, d = e - h * a.dim;
            float v;
            if (d >= a.rot_dims) v = load_as_f32(a.x[which], a.dtype, in + e);
            else {
                const int i = d < half ? d : d - half;
                float s, c;
                sincosf((float)pos * a.inv_freq[i], &s, &c);
                const float u = load_as_f32(a.x[which], a.dtype, in + h * a.dim + i);
                const float w = load_as_f32(a.x[which], a.dtype, in + h * a.dim + i + half);
                v = d < half ? u * c - w * s : w * c + u * s;
            }
            o[e] = v * a.scale[which];
        }
    }
}

LLME_API int llme_rotate(const LlmeRotateArgs* args, cudaStream_t stream) {
    const LlmeRotateArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (!a.positions || (a.rot_dims > 0 && !a.inv_freq)) LLME_REFUSE("rotate: null pointer");
    if (a.rot_dims < 0 || a.rot_dims % 2 || a.rot_dims > a.dim) LLME_REFUSE("rotate: %d rotated coordinates of %d need an even count", a.rot_dims, a.dim);
    if (a.dtype != LLME_F32 && a.dtype != LLME_BF16) LLME_REFUSE("rotate: unsupported dtype %d", a.dtype);
    for (int i = 0; i < 2; ++i)
        if (a.x[i] && !a.out[i]) LLME_REFUSE("rotate: no place for a result");
    const int widest = max(a.x[0] ? a.heads[0] : 0, a.x[1] ? a.heads[1] : 0) * a.dim;
    const int threads = widest >= 1024 ? 256 : 128;
    llme_launch(rotate_kernel, dim3(a.tokens), dim3(threads), 0, stream, a);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- the recurrence
// One warp owns one column of a head's state (the n values that meet one coordinate of v): lane l holds S[l + 32 r], r < R,
// in registers for all tokens of the request's portion; a token costs R multiply-adds for the update, R for the output and
// one sum over the lanes.  Columns are independent, so no warp waits for another.  A block takes WARPS columns of one
// (request, head); the state is stored column by column, so a warp's loads and stores of it are contiguous.
template <int R>
__global__ void __launch_bounds__(256) recurrence_kernel(LlmeRecurrenceArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int j = blockIdx.x * warps + (threadIdx.x >> 5);          // column: coordinate of v
    const int h = blockIdx.y, r = blockIdx.z;
    if (j >= a.p) return;
    const int n = a.n, p = a.p;
    const int first = a.cu_q_lens[r], last = a.cu_q_lens[r + 1];
    const int g = h / (a.heads / a.qk_groups);
    float* st = a.state + (size_t)a.state_slots[r] * a.state_stride + ((size_t)h * p + j) * n;
    float S[R];
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = lane + 32 * i < n ? st[lane + 32 * i] : 0.0f;
    const float fixed = a.gate == 0 ? a.decay[h] : 0.0f;
    const float rate = a.gate == 1 ? -expf(a.a_log[h]) : 0.0f;
    const float bias = a.gate == 1 && a.dt_bias ? a.dt_bias[h] : 0.0f;
    const float skip = a.skip ? a.skip[h] : 0.0f;
    for (int t = first; t < last; ++t) {
        const float* q = a.q + (size_t)t * a.ldq + (size_t)g * n;
        const float* k = a.k + (size_t)t * a.ldk + (size_t)g * n;
        const float v = load_as_f32(a.v, a.v_dtype, (size_t)t * a.ldv + (size_t)h * p + j);
        float decay = fixed, step = 1.0f;
        if (a.gate == 1) {
            step = softplus32(load_as_f32(a.dt, a.dt_dtype, (size_t)t * a.lddt + h) + bias);
            decay = expf(rate * step);
        }
        const float sv = step;
        float y = 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int e = lane + 32 * i;
            if (e < n) {
                S[i] = fmaf(decay, S[i], (sv * k[e]) * v);
                y = fmaf(S[i], q[e], y);
            }
        }
        y = warp_sum(y);
        if (lane == 0) a.out[(size_t)t * a.ldo + (size_t)h * p + j] = y + skip * v;
    }
#pragma unroll
    for (int i = 0; i < R; ++i)
        if (lane + 32 * i < n) st[lane + 32 * i] = S[i];
}

LLME_API int llme_recurrence(const LlmeRecurrenceArgs* args, cudaStream_t stream) {
    const LlmeRecurrenceArgs& a = *args;
    if (a.requests <= 0) return 0;
    if (!a.q || !a.k || !a.v || !a.state || !a.out || !a.cu_q_lens || !a.state_slots) LLME_REFUSE("recurrence: null pointer");
    if (a.heads <= 0 || a.n <= 0 || a.p <= 0 || a.qk_groups <= 0 || a.heads % a.qk_groups) LLME_REFUSE("recurrence: %d heads in %d groups", a.heads, a.qk_groups);
    if (a.gate == 0 ? !a.decay : (a.gate != 1 || !a.dt || !a.a_log)) LLME_REFUSE("recurrence: gate %d lacks its constants", a.gate);
    if (a.n > 512) LLME_REFUSE("recurrence: a state of %d rows per column, this build takes up to 512", a.n);
    if (a.heads > 65535 || a.requests > 65535) LLME_REFUSE("recurrence: too many heads or requests for one launch");
    const int warps = a.p >= 8 ? 8 : a.p;
    const dim3 grid((a.p + warps - 1) / warps, a.heads, a.requests), block(32 * warps);
    if (a.n <= 32) llme_launch(recurrence_kernel<1>, grid, block, 0, stream, a);
    else if (a.n <= 64) llme_launch(recurrence_kernel<2>, grid, block, 0, stream, a);
    else if (a.n <= 128) llme_launch(recurrence_kernel<4>, grid, block, 0, stream, a);
    else if (a.n <= 256) llme_launch(recurrence_kernel<8>, grid, block, 0, stream, a);
    else llme_launch(recurrence_kernel<16>, grid, block, 0, stream, a);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- grouped RMS norm with a silu gate
template <typename T>
__global__ void gated_norm_kernel(LlmeGatedNormArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int groups = a.cols / a.group;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);      // (token, group)
    if (item >= (long long)a.tokens * groups) return;
    const int t = (int)(item / groups), c0 = (int)(item - (long long)t * groups) * a.group;
    const float* y = a.y + (size_t)t * a.ldy + c0;
    const T* g = (const T*)a.gate + (size_t)t * a.ldg + c0;
    T* o = (T*)a.out + (size_t)t * a.ldo + c0;
    float ss = 0.0f;
    for (int c = lane; c < a.group; c += 32) {
        const float u = a.gate_first ? y[c] * silu32(to_f32(g[c])) : y[c];
        ss += u * u;
    }
    const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)a.group + a.eps);
    for (int c = lane; c < a.group; c += 32) {
        const float gate = silu32(to_f32(g[c]));
        float u = (a.gate_first ? y[c] * gate : y[c]) * rinv;
        if (a.weight) u *= a.weight[c0 + c];
        if (!a.gate_first) u *= gate;
        o[c] = from_f32<T>(u * a.scale);
    }
}

LLME_API int llme_gated_norm(const LlmeGatedNormArgs* args, cudaStream_t stream) {
    const LlmeGatedNormArgs& a = *args;
    if (a.tokens <= 0 || a.cols <= 0) return 0;
    if (!a.y || !a.gate || !a.out) LLME_REFUSE("gated_norm: null pointer");
    if (a.group <= 0 || a.cols % a.group) LLME_REFUSE("gated_norm: %d columns are not whole groups of %d", a.cols, a.group);
    if (!(a.eps > 0.0f)) LLME_REFUSE("gated_norm: eps must be positive");
    const int warps = 4;
    const long long items = (long long)a.tokens * (a.cols / a.group);
    const dim3 grid((unsigned)((items + warps - 1) / warps)), block(32 * warps);
    if (a.dtype == LLME_F32) llme_launch(gated_norm_kernel<float>, grid, block, 0, stream, a);
    else if (a.dtype == LLME_BF16) llme_launch(gated_norm_kernel<__nv_bfloat16>, grid, block, 0, stream, a);
    else LLME_REFUSE("gated_norm: unsupported dtype %d", a.dtype);
    LLME_LAUNCH_STATUS();
}

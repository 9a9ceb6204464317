// Layers that carry a state of fixed size per request instead of a cache that grows: a short causal convolution per
// channel, the rotation of queries and keys into 32-bit, a linear recurrence with a decaying matrix state per head
// (linear attention with a fixed decay per head; a selective state space whose decay and step come with every token), and
// the grouped RMS norm with a silu gate that follows such a recurrence.  Everything that enters the recurrence is 32-bit,
// and so is the state.  A request's tokens are taken in their order; only where a long portion is cut into pieces (by the
// step's size) does the order of the state's sums change, so what a token gets depends on how its prompt was cut into steps
// and on what else the step holds by 32-bit rounding and no more.
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

// The same for a number of taps known when compiling: a thread takes four channels at once, all their inputs and weights on
// their way before the first sum (the sums in the order of the kernel above).
template <int K>
__global__ void short_conv_taps_kernel(LlmeShortConvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int r = row_of_token(a.cu_q_lens, a.requests, t);
    const int i = t - a.cu_q_lens[r];
    const float* st = a.state + (size_t)a.state_slots[r] * a.state_stride;
    const int stride = gridDim.y * blockDim.x;
    for (int c0 = blockIdx.y * blockDim.x + threadIdx.x; c0 < a.channels; c0 += 4 * stride) {
        float x[4][K], w[4][K], y[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int c = c0 + m * stride;
            const bool ok = c < a.channels;
            y[m] = ok && a.bias ? a.bias[c] : 0.0f;
#pragma unroll
            for (int j = 0; j < K; ++j) {
                const int src = i - j;
                x[m][j] = !ok ? 0.0f : src >= 0 ? load_as_f32(a.x, a.x_dtype, (size_t)(t - j) * a.ldx + c) : st[(size_t)(K - 1 + src) * a.channels + c];
                w[m][j] = ok ? a.w[(size_t)c * K + (K - 1 - j)] : 0.0f;
            }
        }
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int c = c0 + m * stride;
#pragma unroll
            for (int j = K - 1; j >= 0; --j) y[m] = fmaf(w[m][j], x[m][j], y[m]);
            if (c < a.channels) a.out[(size_t)t * a.ldo + c] = a.act == 1 ? silu32(y[m]) : y[m];
        }
    }
}

// Prompt portions whose rows allow loads of four channels at once: a thread owns four neighbouring channels and walks over
// CONV_TOKENS tokens of the step, keeping the K - 1 inputs before the present one in registers, so an input is read once (and
// once more by the block that takes the next tokens); where a request begins inside the walk the window is read anew (from the
// request's state).  The sums are those of the kernel above, in its order.
constexpr int CONV_TOKENS = 16;

template <typename T> __device__ __forceinline__ void load_four(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load_four<float>(const float* p, float (&v)[4]) {
    const float4 f = *(const float4*)p;
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
template <> __device__ __forceinline__ void load_four<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 raw = *(const uint2*)p;
    const __nv_bfloat162 lo = *(const __nv_bfloat162*)&raw.x, hi = *(const __nv_bfloat162*)&raw.y;
    v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
}

template <int K, typename T>
__global__ void __launch_bounds__(128) short_conv_walk_kernel(LlmeShortConvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= a.channels) return;
    const int t0 = blockIdx.x * CONV_TOKENS, t1 = min(a.tokens, t0 + CONV_TOKENS);
    float w[4][K], bias[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        bias[m] = a.bias ? a.bias[c + m] : 0.0f;
#pragma unroll
        for (int j = 0; j < K; ++j) w[m][j] = a.w[(size_t)(c + m) * K + (K - 1 - j)];      // w[m][j] meets the input j tokens back
    }
    const T* x = (const T*)a.x;
    float present[CONV_TOKENS][4];                                      // all of the walk's inputs are on their way at once
#pragma unroll
    for (int u = 0; u < CONV_TOKENS; ++u)
        if (t0 + u < t1) load_four<T>(x + (size_t)(t0 + u) * a.ldx + c, present[u]);
    float back[K][4];                                                   // back[j]: the input j tokens before the present one
    int r = row_of_token(a.cu_q_lens, a.requests, t0), begin = a.cu_q_lens[r], end = a.cu_q_lens[r + 1];
    bool fresh = true;
#pragma unroll
    for (int u = 0; u < CONV_TOKENS; ++u) {
        const int t = t0 + u;
        if (t >= t1) break;
        while (t >= end) {                                              // the next request that has tokens
            ++r;
            begin = end;
            end = a.cu_q_lens[r + 1];
            fresh = true;
        }
        const int i = t - begin;
        if (fresh) {
            const float* st = a.state + (size_t)a.state_slots[r] * a.state_stride;
#pragma unroll
            for (int j = 1; j < K; ++j) {
                if (i - j >= 0) load_four<T>(x + (size_t)(t - j) * a.ldx + c, back[j]);
                else load_four<float>(st + (size_t)(K - 1 + i - j) * a.channels + c, back[j]);
            }
            fresh = false;
        }
        float y[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            back[0][m] = present[u][m];
            y[m] = bias[m];
#pragma unroll
            for (int j = K - 1; j >= 0; --j) y[m] = fmaf(w[m][j], back[j][m], y[m]);
            if (a.act == 1) y[m] = silu32(y[m]);
        }
        *(float4*)(a.out + (size_t)t * a.ldo + c) = make_float4(y[0], y[1], y[2], y[3]);
#pragma unroll
        for (int j = K - 1; j > 0; --j)
#pragma unroll
            for (int m = 0; m < 4; ++m) back[j][m] = back[j - 1][m];
    }
}

template <int K>
static void short_conv_walk(const LlmeShortConvArgs& a, cudaStream_t stream) {
    const dim3 grid((a.tokens + CONV_TOKENS - 1) / CONV_TOKENS, (a.channels / 4 + 127) / 128), block(128);
    if (a.x_dtype == LLME_F32) llme_launch(short_conv_walk_kernel<K, float>, grid, block, 0, stream, a);
    else llme_launch(short_conv_walk_kernel<K, __nv_bfloat16>, grid, block, 0, stream, a);
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
        // a thread takes up to four channels of its token, more where the step has too few tokens to fill the GPU otherwise
        const int fill = (592 + a.tokens - 1) / a.tokens, quarter = (pieces + 3) / 4;
        pieces = min(pieces, max(fill, quarter));
        // rows of x, of the output and of the state that start on 16 bytes (8 for bf16 inputs), channels in fours
        const size_t el = a.x_dtype == LLME_F32 ? 4 : 2;
        const bool fours = a.channels % 4 == 0 && (uintptr_t)a.x % (4 * el) == 0 && a.ldx % 4 == 0 && (uintptr_t)a.out % 16 == 0 &&
                           a.ldo % 4 == 0 && (uintptr_t)a.state % 16 == 0 && a.state_stride % 4 == 0;
        if (fours && a.tokens >= 8 * CONV_TOKENS && a.taps >= 2 && a.taps <= 4) {
            if (a.taps == 4) short_conv_walk<4>(a, stream);
            else if (a.taps == 3) short_conv_walk<3>(a, stream);
            else short_conv_walk<2>(a, stream);
            LLME_LAUNCH_STATUS();
        }
        const dim3 grid(a.tokens, pieces < 1 ? 1 : pieces);
        if (a.taps == 4) llme_launch(short_conv_taps_kernel<4>, grid, dim3(threads), 0, stream, a);
        else if (a.taps == 3) llme_launch(short_conv_taps_kernel<3>, grid, dim3(threads), 0, stream, a);
        else if (a.taps == 2) llme_launch(short_conv_taps_kernel<2>, grid, dim3(threads), 0, stream, a);
        else llme_launch(short_conv_kernel, grid, dim3(threads), 0, stream, a);
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
        for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < total; e += gridDim.y * blockDim.x) {
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
    // a step of few tokens spreads a token's columns over several blocks
    const int most = (widest + threads - 1) / threads, fill = (592 + a.tokens - 1) / a.tokens;
    llme_launch(rotate_kernel, dim3(a.tokens, most < fill ? most : fill), dim3(threads), 0, stream, a);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- the recurrence
// Single tokens (and states with fewer than four columns): one warp owns one column of a head's state (the n values that meet
// one coordinate of v): lane l holds S[l + 32 i], i < R, in registers; a token costs R multiply-adds for the update, R for the
// output and one sum over the lanes.  Columns are independent, so no warp waits for another.  A block takes WARPS columns of
// one (request, head); the state is stored column by column, so a warp's loads and stores of it are contiguous.
template <int R>
__global__ void __launch_bounds__(256) recurrence_column_kernel(LlmeRecurrenceArgs a) {
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
    const int vp = a.unit_column ? p - 1 : p;                       // columns that have a v behind them
    for (int t = first; t < last; ++t) {
        const float* q = a.q + (size_t)t * a.ldq + (size_t)g * n;
        const float* k = a.k + (size_t)t * a.ldk + (size_t)g * n;
        const float v = j < vp ? load_as_f32(a.v, a.v_dtype, (size_t)t * a.ldv + (size_t)h * vp + j) : 1.0f;
        float decay = fixed, step = 1.0f;
        if (a.gate == 1) {
            step = softplus32(load_as_f32(a.dt, a.dt_dtype, (size_t)t * a.lddt + h) + bias);
            decay = expf(rate * step);
        } else if (a.gate == 2) {
            decay = a.keep[(size_t)t * a.ld_gates + h];
            step = a.take[(size_t)t * a.ld_gates + h];
        }
        float y = 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int e = lane + 32 * i;
            if (e < n) {
                S[i] = fmaf(decay, S[i], (step * k[e]) * v);
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

// Portions of prompts: a block of eight warps takes 32 neighbouring columns of one (request or piece of it, head), four a warp
// (lane l holds S[R l + i], i < R, of each of its four, so its q and k come from shared memory in one piece).  The block brings q and k of a few tokens at a time into shared memory with
// asynchronous copies, and v, the steps and the decays beside them, while it works on the tokens before: every warp of the
// block needs the same q and k, and no token's operands come from global memory when they are due.  A token costs a warp 4 R
// multiply-adds for the update, 4 R for the output, and six exchanges that sum the four columns over the lanes (each lane
// ending with the sum of one column).
//
// A request with many tokens in the step is cut into pieces of `chunk` tokens that run side by side, in three launches:
// every piece but a request's last starts from zero and leaves E_c, what its tokens alone add to the state, and D_c, the
// product of its decays; then, per state element and in the pieces' order, B_0 = the stored state, B_(c+1) = D_c B_c + E_c
// gives every piece the state it starts from; then every piece runs from B_c, writes its outputs, and the last one stores
// the state.  The sum is the one of the plain walk in another order, all of it 32-bit.
enum { REC_WHOLE = 0, REC_LOCAL = 1, REC_FROM_START = 2 };
constexpr int REC_MIN_CHUNK = 64, REC_COLUMNS = 32;

struct RecPiece { int r, index, pieces, slot; };

// Piece z of the step when every request is cut each `chunk` tokens; `slot` counts the pieces of requests with several.
__device__ __forceinline__ bool rec_find_piece(const int* __restrict__ cu, int requests, int chunk, int z, RecPiece& o) {
    int multi = 0;
    for (int i = 0; i < requests; ++i) {
        const int np = (cu[i + 1] - cu[i] + chunk - 1) / chunk;
        if (z < np) { o.r = i; o.index = z; o.pieces = np; o.slot = multi + z; return true; }
        z -= np;
        if (np > 1) multi += np;
    }
    return false;
}

__device__ __forceinline__ void copy_async_4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Two 32-bit values in one 64-bit register and the packed multiply-add on both (each half rounds as fmaf does).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

template <int R> struct RecTile {
    static constexpr int TOKENS = R <= 4 ? 16 : (R == 8 ? 8 : 4);       // tokens in shared memory at a time, twice
    static constexpr int ROW = 32 * R;                                   // n rounded up
    static constexpr int V_EACH = (TOKENS * REC_COLUMNS + 255) / 256;    // values of v a thread fetches
    float q[2][TOKENS][ROW], k[2][TOKENS][ROW], v[2][TOKENS][REC_COLUMNS], step[2][TOKENS], decay[2][TOKENS];
    float sums[8][TOKENS][16];                                         // per warp and token: four partial sums of each of four columns
};

template <int R, bool LOCAL>
__global__ void __launch_bounds__(256, R <= 4 ? 3 : 1) recurrence_tile_kernel(LlmeRecurrenceArgs a, int pass, int chunk, int slots, int vec) {
    using Tile = RecTile<R>;
    constexpr int TT = Tile::TOKENS, ROW = Tile::ROW, V_EACH = Tile::V_EACH;
    __shared__ __align__(16) Tile sm;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int jb = blockIdx.x * REC_COLUMNS, j0 = jb + 4 * warp;        // the block's and the warp's first column
    const int h = blockIdx.y, n = a.n, p = a.p;
    RecPiece pc = {(int)blockIdx.z, 0, 1, 0};
    if (pass != REC_WHOLE && !rec_find_piece(a.cu_q_lens, a.requests, chunk, blockIdx.z, pc)) return;
    const bool last_piece = pc.index == pc.pieces - 1;
    if (LOCAL && last_piece) return;
    int first = a.cu_q_lens[pc.r], last = a.cu_q_lens[pc.r + 1];
    if (pass != REC_WHOLE) {
        first += pc.index * chunk;
        last = min(last, first + chunk);
    }
    const bool active = j0 < p;
    const size_t hpn = (size_t)a.heads * p * n, column = ((size_t)h * p + j0) * n;
    float* kept = a.state + (size_t)a.state_slots[pc.r] * a.state_stride + column;
    float* mine = pc.pieces > 1 ? a.scratch + (size_t)pc.slot * hpn + column : nullptr;
    const float* from = LOCAL || !active ? nullptr : (mine ? mine : kept);
    f32x2 S[2][R];                                                     // columns 0 | 1 and 2 | 3, packed
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const bool row = from && lane * R + i < n;
            S[c][i] = pack2(row && j0 + 2 * c < p ? from[(size_t)(2 * c) * n + lane * R + i] : 0.0f,
                            row && j0 + 2 * c + 1 < p ? from[(size_t)(2 * c + 1) * n + lane * R + i] : 0.0f);
        }
    const int g = h / (a.heads / a.qk_groups);
    const float fixed = a.gate == 0 ? a.decay[h] : 0.0f;
    const float rate = a.gate == 1 ? -expf(a.a_log[h]) : 0.0f;
    const float bias = a.gate == 1 && a.dt_bias ? a.dt_bias[h] : 0.0f;
    const float skip = a.skip ? a.skip[h] : 0.0f;
    const float* qg = a.q + (size_t)g * n;
    const float* kg = a.k + (size_t)g * n;

    const int vp = a.unit_column ? p - 1 : p;                           // columns that have a v behind them
    float v_next[V_EACH], dt_next = 0.0f, keep_next = 1.0f;
    // Sends for the tokens t0 .. t0 + TT - 1: q and k straight into buffer b, v and dt into registers for now.
    auto fetch = [&](int t0, int b) {
        if (vec) {
            for (int idx = tid; idx < TT * (ROW / 4); idx += 256) {
                const int u = idx / (ROW / 4), e = (idx % (ROW / 4)) * 4, t = t0 + u;
                if (e >= n) continue;
                if (t < last) {
                    copy_async_16(&sm.q[b][u][e], qg + (size_t)t * a.ldq + e);
                    copy_async_16(&sm.k[b][u][e], kg + (size_t)t * a.ldk + e);
                } else {
                    *(float4*)&sm.q[b][u][e] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    *(float4*)&sm.k[b][u][e] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
        } else {
            for (int idx = tid; idx < TT * ROW; idx += 256) {
                const int u = idx / ROW, e = idx % ROW, t = t0 + u;
                if (e >= n) continue;
                if (t < last) {
                    copy_async_4(&sm.q[b][u][e], qg + (size_t)t * a.ldq + e);
                    copy_async_4(&sm.k[b][u][e], kg + (size_t)t * a.ldk + e);
                } else sm.q[b][u][e] = sm.k[b][u][e] = 0.0f;
            }
        }
#pragma unroll
        for (int m = 0; m < V_EACH; ++m) {
            const int idx = tid + 256 * m, u = idx / REC_COLUMNS, c = idx % REC_COLUMNS, t = t0 + u;
            v_next[m] = u < TT && t < last && jb + c < p
                            ? (jb + c < vp ? load_as_f32(a.v, a.v_dtype, (size_t)t * a.ldv + (size_t)h * vp + jb + c) : 1.0f) : 0.0f;
        }
        dt_next = tid < TT && a.gate == 1 && t0 + tid < last ? load_as_f32(a.dt, a.dt_dtype, (size_t)(t0 + tid) * a.lddt + h) : 0.0f;
        if (tid < TT && a.gate == 2 && t0 + tid < last) {
            dt_next = a.take[(size_t)(t0 + tid) * a.ld_gates + h];
            keep_next = a.keep[(size_t)(t0 + tid) * a.ld_gates + h];
        }
    };
    // Completes buffer b; a token past the end gets what changes nothing: q = k = v = 0, step 0, decay 1.
    auto land = [&](int t0, int b) {
#pragma unroll
        for (int m = 0; m < V_EACH; ++m) {
            const int idx = tid + 256 * m, u = idx / REC_COLUMNS, c = idx % REC_COLUMNS;
            if (u < TT) sm.v[b][u][c] = v_next[m];
        }
        if (tid < TT) {
            float st = 0.0f, dc = 1.0f;
            if (t0 + tid < last) {
                st = a.gate == 1 ? softplus32(dt_next + bias) : (a.gate == 2 ? dt_next : 1.0f);
                dc = a.gate == 1 ? expf(rate * st) : (a.gate == 2 ? keep_next : fixed);
            }
            sm.step[b][tid] = st;
            sm.decay[b][tid] = dc;
        }
        copy_async_wait();
        __syncthreads();
    };

    const int tiles = (last - first + TT - 1) / TT;
    if (n < ROW)                                                       // the rows' padding stays zero
        for (int idx = tid; idx < 2 * TT * ROW; idx += 256)
            if (idx % ROW >= n) (&sm.q[0][0][0])[idx] = (&sm.k[0][0][0])[idx] = 0.0f;
    if (tiles > 0) {
        const int t0 = first + (LOCAL ? tiles - 1 : 0) * TT;
        fetch(t0, 0);
        land(t0, 0);
    }
    // A piece's own addition to the state is taken from its last token backwards: E = sum_u (s_u prod_(u' > u) a_u') k_u v_u^T,
    // one multiply-add an element and token, with `total` the product of the decays of the tokens behind.
    float total = 1.0f;
    for (int i = 0; i < tiles; ++i) {
        const int b = i & 1, tile = LOCAL ? tiles - 1 - i : i, t0 = first + tile * TT;
        const int next = first + (LOCAL ? tile - 1 : tile + 1) * TT;
        if (i + 1 < tiles) fetch(next, b ^ 1);
        if (active && LOCAL) {
#pragma unroll
            for (int u = TT - 1; u >= 0; --u) {
                const float w = sm.step[b][u] * total;
                const float4 v4 = *(const float4*)&sm.v[b][u][4 * warp];
                const f32x2 v01 = pack2(v4.x, v4.y), v23 = pack2(v4.z, v4.w);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float kw = w * sm.k[b][u][lane * R + r];
                    const f32x2 kw2 = pack2(kw, kw);
                    S[0][r] = fma2(kw2, v01, S[0][r]);
                    S[1][r] = fma2(kw2, v23, S[1][r]);
                }
                total *= sm.decay[b][u];
            }
        } else if (active) {
#pragma unroll
            for (int u = 0; u < TT; ++u) {
                const float step = sm.step[b][u], decay = sm.decay[b][u];
                const float4 v4 = *(const float4*)&sm.v[b][u][4 * warp];
                const f32x2 v01 = pack2(v4.x, v4.y), v23 = pack2(v4.z, v4.w), decay2 = pack2(decay, decay);
                f32x2 y01 = pack2(0.0f, 0.0f), y23 = y01;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float qi = sm.q[b][u][lane * R + r], ks = step * sm.k[b][u][lane * R + r];
                    const f32x2 qi2 = pack2(qi, qi), ks2 = pack2(ks, ks);
                    S[0][r] = fma2(decay2, S[0][r], mul2(ks2, v01));      // S = a S + (s k) v, as the single-token kernel rounds it
                    S[1][r] = fma2(decay2, S[1][r], mul2(ks2, v23));
                    y01 = fma2(S[0][r], qi2, y01);
                    y23 = fma2(S[1][r], qi2, y23);
                }
                float y[4];
                unpack2(y01, y[0], y[1]);
                unpack2(y23, y[2], y[3]);
                // lanes 16..31 take over columns 2 and 3, then of each half the lanes with bit 3 set the odd column; after one
                // more exchange lanes 8 c .. 8 c + 3 hold four parts of column c, which go to shared memory
                const bool upper = lane & 16, odd = lane & 8;
                const float k0 = (upper ? y[2] : y[0]) + __shfl_xor_sync(0xffffffffu, upper ? y[0] : y[2], 16);
                const float k1 = (upper ? y[3] : y[1]) + __shfl_xor_sync(0xffffffffu, upper ? y[1] : y[3], 16);
                float sum = (odd ? k1 : k0) + __shfl_xor_sync(0xffffffffu, odd ? k0 : k1, 8);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if ((lane & 4) == 0) sm.sums[warp][u][(lane >> 3) * 4 + (lane & 3)] = sum;
            }
            __syncwarp();
            for (int o = lane; o < TT * 4; o += 32) {                  // an output a lane: (token, column)
                const int u = o >> 2, col = o & 3, t = t0 + u;
                const float4 part = *(const float4*)&sm.sums[warp][u][col * 4];
                if (t < last && j0 + col < p)
                    a.out[(size_t)t * a.ldo + (size_t)h * p + j0 + col] = ((part.x + part.y) + (part.z + part.w)) + skip * sm.v[b][u][4 * warp + col];
            }
            __syncwarp();
        }
        if (i + 1 < tiles) land(next, b ^ 1);
    }
    float* to = !active ? nullptr : LOCAL ? mine : (pass == REC_WHOLE || last_piece ? kept : nullptr);
    if (to) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < R; ++i) {
                float lo, hi;
                unpack2(S[c][i], lo, hi);
                if (j0 + 2 * c < p && lane * R + i < n) to[(size_t)(2 * c) * n + lane * R + i] = lo;
                if (j0 + 2 * c + 1 < p && lane * R + i < n) to[(size_t)(2 * c + 1) * n + lane * R + i] = hi;
            }
    }
    if (LOCAL && j0 == 0 && lane == 0) a.scratch[(size_t)slots * hpn + (size_t)pc.slot * a.heads + h] = total;
}

// The second of the three launches: one thread per element of a request's state walks over the request's pieces.
__global__ void recurrence_join_kernel(LlmeRecurrenceArgs a, int chunk, int slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y;
    const int pieces = (a.cu_q_lens[r + 1] - a.cu_q_lens[r] + chunk - 1) / chunk;
    if (pieces < 2) return;
    int base = 0;
    for (int i = 0; i < r; ++i) {
        const int np = (a.cu_q_lens[i + 1] - a.cu_q_lens[i] + chunk - 1) / chunk;
        if (np > 1) base += np;
    }
    const size_t hpn = (size_t)a.heads * a.p * a.n, pn = (size_t)a.p * a.n;
    const float* kept = a.state + (size_t)a.state_slots[r] * a.state_stride;
    const float* products = a.scratch + (size_t)slots * hpn + (size_t)base * a.heads;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < hpn; e += (size_t)gridDim.x * blockDim.x) {
        const int h = (int)(e / pn);
        float* at = a.scratch + (size_t)base * hpn + e;
        float S = kept[e];
        int c = 0;
        for (; c + 4 < pieces; c += 4, at += 4 * hpn) {                  // four pieces' loads are on their way at a time
            float added[4], product[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                added[m] = at[(size_t)m * hpn];
                product[m] = products[(size_t)(c + m) * a.heads + h];
            }
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                at[(size_t)m * hpn] = S;
                S = fmaf(product[m], S, added[m]);
            }
        }
        for (; c + 1 < pieces; ++c, at += hpn) {
            const float added = *at;
            *at = S;
            S = fmaf(products[(size_t)c * a.heads + h], S, added);
        }
        *at = S;
    }
}

template <bool LOCAL>
static void recurrence_tiles(const LlmeRecurrenceArgs& a, dim3 grid, int pass, int chunk, int slots, int vec, cudaStream_t stream) {
    const dim3 block(256);
    if (a.n <= 32) llme_launch(recurrence_tile_kernel<1, LOCAL>, grid, block, 0, stream, a, pass, chunk, slots, vec);
    else if (a.n <= 64) llme_launch(recurrence_tile_kernel<2, LOCAL>, grid, block, 0, stream, a, pass, chunk, slots, vec);
    else if (a.n <= 128) llme_launch(recurrence_tile_kernel<4, LOCAL>, grid, block, 0, stream, a, pass, chunk, slots, vec);
    else if (a.n <= 256) llme_launch(recurrence_tile_kernel<8, LOCAL>, grid, block, 0, stream, a, pass, chunk, slots, vec);
    else llme_launch(recurrence_tile_kernel<16, LOCAL>, grid, block, 0, stream, a, pass, chunk, slots, vec);
}

// The chunk a step of `tokens` tokens whose longest request brings `max_len` is cut by, with room for `slots` piece states
// (requests of several pieces have fewer than 2 tokens / chunk pieces together); 0: every request is walked whole.  A piece's
// first tile and its state are waited for, so pieces are no shorter than it takes to give the GPU's 148 SMs, 3 blocks each,
// four rounds of blocks (`blocks` of them work on one piece).
static int recurrence_chunk(int tokens, int max_len, long long slots, long long blocks) {
    if (slots < 4 || max_len <= REC_MIN_CHUNK) return 0;
    long long chunk = (2LL * tokens + slots - 1) / slots;
    if (chunk < REC_MIN_CHUNK) chunk = REC_MIN_CHUNK;
    const long long pieces = (4 * 3 * 148 + blocks - 1) / blocks, fill = tokens / pieces / 32 * 32;
    if (chunk < fill) chunk = fill;
    chunk = (chunk + 31) / 32 * 32;
    return chunk >= max_len ? 0 : (int)chunk;
}

LLME_API int llme_recurrence(const LlmeRecurrenceArgs* args, cudaStream_t stream) {
    const LlmeRecurrenceArgs& a = *args;
    if (a.requests <= 0) return 0;
    if (!a.q || !a.k || !a.v || !a.state || !a.out || !a.cu_q_lens || !a.state_slots) LLME_REFUSE("recurrence: null pointer");
    if (a.heads <= 0 || a.n <= 0 || a.p <= 0 || a.qk_groups <= 0 || a.heads % a.qk_groups) LLME_REFUSE("recurrence: %d heads in %d groups", a.heads, a.qk_groups);
    if (a.gate == 0 ? !a.decay : a.gate == 1 ? (!a.dt || !a.a_log) : (a.gate != 2 || !a.keep || !a.take))
        LLME_REFUSE("recurrence: gate %d lacks its constants", a.gate);
    if (a.unit_column && (a.p < 2 || a.skip)) LLME_REFUSE("recurrence: a column without v stands beside others and has no skip");
    if (a.n > 512) LLME_REFUSE("recurrence: a state of %d rows per column, this build takes up to 512", a.n);
    if (a.heads > 65535 || a.requests > 65535) LLME_REFUSE("recurrence: too many heads or requests for one launch");
    if (a.max_len <= 1 || a.p < 4) {                                    // single tokens, or too few columns for four a warp
        const int warps = a.p >= 8 ? 8 : a.p;
        const dim3 grid((a.p + warps - 1) / warps, a.heads, a.requests), block(32 * warps);
        if (a.n <= 32) llme_launch(recurrence_column_kernel<1>, grid, block, 0, stream, a);
        else if (a.n <= 64) llme_launch(recurrence_column_kernel<2>, grid, block, 0, stream, a);
        else if (a.n <= 128) llme_launch(recurrence_column_kernel<4>, grid, block, 0, stream, a);
        else if (a.n <= 256) llme_launch(recurrence_column_kernel<8>, grid, block, 0, stream, a);
        else llme_launch(recurrence_column_kernel<16>, grid, block, 0, stream, a);
        LLME_LAUNCH_STATUS();
    }
    const long long hpn = (long long)a.heads * a.p * a.n;
    const long long slots = a.scratch ? a.scratch_floats / (hpn + a.heads) : 0;
    const int chunk = recurrence_chunk(a.tokens, a.max_len, slots, (long long)((a.p + REC_COLUMNS - 1) / REC_COLUMNS) * a.heads);
    // 16-byte copies where every row of q and k starts on such a boundary
    const int vec = ((uintptr_t)a.q % 16 == 0 && (uintptr_t)a.k % 16 == 0 && a.ldq % 4 == 0 && a.ldk % 4 == 0 && a.n % 4 == 0) ? 1 : 0;
    dim3 grid((a.p + REC_COLUMNS - 1) / REC_COLUMNS, a.heads, a.requests);
    if (!chunk) {
        recurrence_tiles<false>(a, grid, REC_WHOLE, 0, 0, vec, stream);
        LLME_LAUNCH_STATUS();
    }
    const long long most = (long long)a.tokens / chunk + a.requests;     // no step has more pieces
    if (most > 65535) LLME_REFUSE("recurrence: %lld pieces are too many for one launch", most);
    grid.z = (unsigned)most;
    recurrence_tiles<true>(a, grid, REC_LOCAL, chunk, (int)slots, vec, stream);
    const long long blocks = (hpn + 255) / 256;
    llme_launch(recurrence_join_kernel, dim3((unsigned)(blocks < 1024 ? blocks : 1024), a.requests), dim3(256), 0, stream, a, chunk, (int)slots);
    recurrence_tiles<false>(a, grid, REC_FROM_START, chunk, (int)slots, vec, stream);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- exponential gates with a running maximum
// One block per (request, head), GATE_TILE tokens at a time: every thread forms the two log gates of its token (the
// transcendental part, side by side, into shared memory), one thread walks the running maxima of the tile in the tokens' order
// (an addition and a maximum a token, operands from shared memory), and every thread forms its token's three outputs.  The walk
// is the plain one, so a token's values do not depend on how its request was cut into steps.  A step of single tokens takes one
// warp per block.
__device__ __forceinline__ float log_sigmoid32(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

constexpr int GATE_TILE = 256;

__global__ void exp_gates_kernel(LlmeExpGatesArgs a) {
    __shared__ __align__(16) float ga[GATE_TILE], gb[GATE_TILE];
    __shared__ float mx[GATE_TILE + 8];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, r = blockIdx.y, tile = blockDim.x;
    const int first = a.cu_q_lens[r], last = a.cu_q_lens[r + 1];
    if (last <= first) return;                                      // (uniform over the block)
    float* kept = a.state + (size_t)a.state_slots[r] * a.state_stride + h;
    if (threadIdx.x == 0) mx[0] = *kept;
    for (int t0 = first; t0 < last; t0 += tile) {
        const int t = t0 + threadIdx.x, count = min(tile, last - t0);
        float va = 0.0f, vb = 0.0f;
        if (t < last) {
            va = a.i_pre[(size_t)t * a.ld_pre + h];
            vb = a.f_pre[(size_t)t * a.ld_pre + h];
            if (a.cap > 0.0f) {
                va = a.cap * tanhf(va / a.cap);
                vb = a.cap * tanhf(vb / a.cap);
            }
            vb = log_sigmoid32(vb);
        }
        // behind the step's last token stands what changes nothing: max(0 + M, -inf) = M
        ga[threadIdx.x] = t < last ? va : -INFINITY;
        gb[threadIdx.x] = t < last ? vb : 0.0f;
        __syncthreads();
        if (threadIdx.x == 0) {
            // eight tokens' operands go to registers at once, so that the walk itself waits for no load: an addition and
            // a maximum a token.  mx[u]: the maximum before token u, mx[u + 1]: behind it.
            float M = mx[0];
#pragma unroll 2
            for (int u0 = 0; u0 < count; u0 += 8) {
                const float4 a0 = *(const float4*)&ga[u0], a1 = *(const float4*)&ga[u0 + 4];
                const float4 b0 = *(const float4*)&gb[u0], b1 = *(const float4*)&gb[u0 + 4];
                const float va8[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float vb8[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                float r8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    M = fmaxf(vb8[i] + M, va8[i]);
                    r8[i] = M;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) mx[u0 + i + 1] = r8[i];
            }
        }
        __syncthreads();
        const float before = mx[threadIdx.x < count ? threadIdx.x : 0], after = mx[threadIdx.x < count ? threadIdx.x + 1 : 0];
        const float carried = mx[count];
        __syncthreads();
        if (threadIdx.x == 0) mx[0] = carried;
        if (t < last) {
            a.keep[(size_t)t * a.ld_out + h] = expf(vb + before - after);
            a.take[(size_t)t * a.ld_out + h] = expf(va - after);
            a.floor[(size_t)t * a.ld_out + h] = expf(-after);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *kept = mx[0];
}

LLME_API int llme_exp_gates(const LlmeExpGatesArgs* args, int max_len, cudaStream_t stream) {
    const LlmeExpGatesArgs& a = *args;
    if (a.requests <= 0 || a.heads <= 0) return 0;
    if (!a.i_pre || !a.f_pre || !a.state || !a.keep || !a.take || !a.floor || !a.cu_q_lens || !a.state_slots) LLME_REFUSE("exp_gates: null pointer");
    if (a.cap < 0.0f) LLME_REFUSE("exp_gates: a negative cap");
    if (a.requests > 65535) LLME_REFUSE("exp_gates: too many requests for one launch");
    const int threads = max_len <= 32 ? 32 : (max_len <= 128 ? 128 : GATE_TILE);
    llme_launch(exp_gates_kernel, dim3(a.heads, a.requests), dim3(threads), 0, stream, a);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- grouped RMS norm with a silu gate
__device__ __forceinline__ float gate32(float z, int act) { return act == 1 ? 1.0f / (1.0f + expf(-z)) : silu32(z); }

template <typename T>
__global__ void gated_norm_kernel(LlmeGatedNormArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int groups = a.cols / a.group;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);      // (token, group)
    if (item >= (long long)a.tokens * groups) return;
    const int t = (int)(item / groups), gi = (int)(item - (long long)t * groups), c0 = gi * a.group;
    const float* y = a.y + (size_t)t * a.ldy + (a.floor ? c0 + gi : c0);       // with a floor every group of y is one value wider
    const T* g = (const T*)a.gate + (size_t)t * a.ldg + c0;
    T* o = (T*)a.out + (size_t)t * a.ldo + c0;
    const float den = a.floor ? fmaxf(fabsf(y[a.group]), a.floor[(size_t)t * a.ld_floor + gi]) + a.den_eps : 1.0f;
    float ss = 0.0f;
    for (int c = lane; c < a.group; c += 32) {
        const float yc = a.floor ? y[c] / den : y[c];
        const float u = a.gate_first ? yc * gate32(to_f32(g[c]), a.gate_act) : yc;
        ss += u * u;
    }
    const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)a.group + a.eps);
    for (int c = lane; c < a.group; c += 32) {
        const float gate = gate32(to_f32(g[c]), a.gate_act);
        const float yc = a.floor ? y[c] / den : y[c];
        float u = (a.gate_first ? yc * gate : yc) * rinv;
        if (a.weight) u *= a.weight[c0 + c];
        if (!a.gate_first) u *= gate;
        o[c] = from_f32<T>(u * a.scale);
    }
}

// Groups of more than 128 and up to 1,024 columns: a block per (token, group), a thread for every eight columns (whole warps),
// keeps its values in registers between the sum of squares and the output, so y and the gate are read once and all loads are on
// their way together.
template <typename T>
__global__ void __launch_bounds__(128) gated_norm_block_kernel(LlmeGatedNormArgs a) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int groups = a.cols / a.group;
    const int t = blockIdx.x / groups, gi = blockIdx.x - t * groups, c0 = gi * a.group;
    const float* y = a.y + (size_t)t * a.ldy + (a.floor ? c0 + gi : c0);
    const T* g = (const T*)a.gate + (size_t)t * a.ldg + c0;
    T* o = (T*)a.out + (size_t)t * a.ldo + c0;
    float u[8], gate[8], ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + blockDim.x * i;
        u[i] = c < a.group ? y[c] : 0.0f;
        gate[i] = c < a.group ? to_f32(g[c]) : 0.0f;
    }
    // (the normaliser and its floor are asked for with the row's values, not before them)
    const float den = a.floor ? fmaxf(fabsf(y[a.group]), a.floor[(size_t)t * a.ld_floor + gi]) + a.den_eps : 1.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (a.floor) u[i] = u[i] / den;
        gate[i] = gate32(gate[i], a.gate_act);
        if (a.gate_first) u[i] *= gate[i];
        ss += u[i] * u[i];
    }
    const float rinv = 1.0f / sqrtf(block_sum(ss, red) / (float)a.group + a.eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + blockDim.x * i;
        if (c >= a.group) continue;
        float v = u[i] * rinv;
        if (a.weight) v *= a.weight[c0 + c];
        if (!a.gate_first) v *= gate[i];
        o[c] = from_f32<T>(v * a.scale);
    }
}

LLME_API int llme_gated_norm(const LlmeGatedNormArgs* args, cudaStream_t stream) {
    const LlmeGatedNormArgs& a = *args;
    if (a.tokens <= 0 || a.cols <= 0) return 0;
    if (!a.y || !a.gate || !a.out) LLME_REFUSE("gated_norm: null pointer");
    if (a.group <= 0 || a.cols % a.group) LLME_REFUSE("gated_norm: %d columns are not whole groups of %d", a.cols, a.group);
    if (!(a.eps > 0.0f)) LLME_REFUSE("gated_norm: eps must be positive");
    const long long items = (long long)a.tokens * (a.cols / a.group);
    if (a.group > 128 && a.group <= 1024 && items < (1LL << 31) && (a.dtype == LLME_F32 || a.dtype == LLME_BF16)) {
        const dim3 block(((a.group + 7) / 8 + 31) / 32 * 32);
        if (a.dtype == LLME_F32) llme_launch(gated_norm_block_kernel<float>, dim3((unsigned)items), block, 0, stream, a);
        else llme_launch(gated_norm_block_kernel<__nv_bfloat16>, dim3((unsigned)items), block, 0, stream, a);
        LLME_LAUNCH_STATUS();
    }
    const int warps = 4;
    const dim3 grid((unsigned)((items + warps - 1) / warps)), block(32 * warps);
    if (a.dtype == LLME_F32) llme_launch(gated_norm_kernel<float>, grid, block, 0, stream, a);
    else if (a.dtype == LLME_BF16) llme_launch(gated_norm_kernel<__nv_bfloat16>, grid, block, 0, stream, a);
    else LLME_REFUSE("gated_norm: unsupported dtype %d", a.dtype);
    LLME_LAUNCH_STATUS();
}

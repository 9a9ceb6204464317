// A mixture of experts: routing (sigmoid scores, the largest few chosen, weights normalised over the chosen; or the
// softmax over the chosen logits alone), the list
// of (token, choice) pairs expert by expert, one product per expert over its pairs (plain form: any sizes, both types,
// 32-bit FMA in a fixed order of k, so that a row never depends on what shares its tile), and the weighted sum of a
// token's pairs in the order of its choices.  The tensor-core form of the grouped product is csrc/moe_tc.cu.
#include "common.cuh"
#include "kernel_args.h"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

// ----------------------------------------------------------------------------- routing
// One warp per token: `top_k` rounds of a warp-wide argmax over the logits not chosen yet (ties: the lower index).
__global__ void moe_route_kernel(LlmeMoeRouteArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= a.tokens) return;
    const float* z = a.logits + (size_t)t * a.ld;
    const int E = a.num_experts;
    unsigned taken = 0;                                   // bit i: this lane's i-th logit (lane + 32 i) is chosen
    float total = 0.0f, first = 0.0f;
    float score[8];
    int chosen[8];
    for (int k = 0; k < a.top_k; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int i = lane, n = 0; i < E; i += 32, ++n) {
            if ((taken >> n) & 1u) continue;
            const float v = z[i];
            if (bi < 0 || v > best) { best = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        if (bi >= 0 && (bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (k == 0) first = best;
        // mode 1: the softmax over the chosen logits alone, relative to the largest of them (the first chosen)
        const float s = a.mode == 1 ? expf(best - first) : 1.0f / (1.0f + expf(-best));
        score[k & 7] = s;
        chosen[k & 7] = bi;
        total += s;
        if (a.top_k > 8 && lane == 0) {                   // more choices than the registers hold: store as they come
            a.experts[(size_t)t * a.top_k + k] = bi;
            a.weights[(size_t)t * a.top_k + k] = s;
        }
    }
    const float norm = a.scale / (a.mode == 1 ? total : total + 1e-20f);
    if (lane == 0) {
        for (int k = 0; k < a.top_k; ++k) {
            const size_t at = (size_t)t * a.top_k + k;
            if (a.top_k <= 8) {
                a.experts[at] = chosen[k];
                a.weights[at] = score[k] * norm;
            } else {
                a.weights[at] *= norm;
            }
            atomicAdd(a.counts + a.experts[at], 1);
        }
    }
}

// One block: offsets from the counts, the pairs placed expert by expert, the counts cleared for the next launch.  The
// order of the pairs inside an expert's range is whatever the atomics give: no result depends on it, since every row
// of a grouped product is computed by itself.
__global__ void moe_order_kernel(LlmeMoeRouteArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int cursor[];                       // [E + 1]
    const int E = a.num_experts, P = a.tokens * a.top_k;
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = at;
            a.offsets[e] = at;
            at += a.counts[e];
        }
        cursor[E] = at;
        a.offsets[E] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < P; i += blockDim.x) a.order[atomicAdd(cursor + a.experts[i], 1)] = i;
    for (int e = threadIdx.x; e < E; e += blockDim.x) a.counts[e] = 0;
}

LLME_API int llme_moe_route(const LlmeMoeRouteArgs* args, cudaStream_t stream) {
    const LlmeMoeRouteArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (!a.logits || !a.experts || !a.weights || !a.offsets || !a.order || !a.counts) LLME_REFUSE("moe_route: null pointer");
    if (a.mode != 0 && a.mode != 1) LLME_REFUSE("moe_route: unknown mode %d", a.mode);
    if (a.num_experts <= 0 || a.num_experts > 1024 || a.top_k <= 0 || a.top_k > a.num_experts)
        LLME_REFUSE("moe_route: %d of %d experts (at most 1024)", a.top_k, a.num_experts);
    const int wpb = 4;
    llme_launch(moe_route_kernel, dim3((a.tokens + wpb - 1) / wpb), dim3(wpb * 32), 0, stream, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(llme_error_buffer(), 512, "%s", cudaGetErrorString(e));
        return (int)e;
    }
    llme_launch(moe_order_kernel, dim3(1), dim3(1024), (size_t)(a.num_experts + 1) * sizeof(int), stream, a);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- one product per expert, plain form
// The row tiles of all experts are numbered one after the other; a block finds the expert of its tile from the offsets.
__device__ __forceinline__ bool find_tile(const int* __restrict__ offsets, int E, int BM, int tile, int* expert, int* first, int* rows) {
    int seen = 0;
    for (int e = 0; e < E; ++e) {
        const int lo = offsets[e], n = offsets[e + 1] - lo;
        const int tiles = (n + BM - 1) / BM;
        if (tile < seen + tiles) {
            const int at = (tile - seen) * BM;
            *expert = e;
            *first = lo + at;
            *rows = n - at < BM ? n - at : BM;
            return true;
        }
        seen += tiles;
    }
    return false;
}

constexpr int GM = 16, GN = 64, GK = 16;

template <typename T, typename W, typename O>
__global__ void __launch_bounds__(256) grouped_linear_kernel(LlmeGroupedArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ int s_tile[3];
    __shared__ int s_src[GM], s_dst[GM];
    __shared__ float xs[GM][GK + 1];
    __shared__ float ws[2][GN][GK + 1];
    if (threadIdx.x == 0) {
        int e = -1, first = 0, rows = 0;
        if (!find_tile(a.offsets, a.num_experts, GM, blockIdx.y, &e, &first, &rows)) e = -1;
        s_tile[0] = e; s_tile[1] = first; s_tile[2] = rows;
    }
    __syncthreads();
    const int e = s_tile[0], first = s_tile[1], rows = s_tile[2];
    if (e < 0) return;
    if (threadIdx.x < GM) {
        const int r = threadIdx.x;
        const int pair = r < rows ? a.order[first + r] : -1;
        s_src[r] = r < rows ? (a.gather ? pair / a.top_k : first + r) : -1;
        s_dst[r] = r < rows ? (a.scatter ? pair : first + r) : -1;
    }
    __syncthreads();
    const int n_out = a.act ? a.n / 2 : a.n;
    const int col0 = blockIdx.x * GN;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;        // row ty, columns tx + 16 c
    const W* w = (const W*)a.w + (size_t)e * a.w_expert;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < a.k; k0 += GK) {
        {
            const int r = threadIdx.x >> 4, kk = threadIdx.x & 15;
            const int src = s_src[r];
            xs[r][kk] = (src >= 0 && k0 + kk < a.k) ? to_f32(((const T*)a.x)[(size_t)src * a.ldx + k0 + kk]) : 0.0f;
        }
        for (int i = threadIdx.x; i < (a.act ? 2 : 1) * GN * GK; i += 256) {
            const int half = i / (GN * GK), c = (i / GK) % GN, kk = i % GK;
            const int row = half * n_out + col0 + c;
            ws[half][c][kk] = (col0 + c < n_out && k0 + kk < a.k) ? to_f32(w[(size_t)row * a.ldw + k0 + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            const float xv = xs[ty][kk];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                acc[0][c] = fmaf(xv, ws[0][tx + 16 * c][kk], acc[0][c]);
                if (a.act) acc[1][c] = fmaf(xv, ws[1][tx + 16 * c][kk], acc[1][c]);
            }
        }
        __syncthreads();
    }
    const int dst = s_dst[ty];
    if (dst < 0) return;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int col = col0 + tx + 16 * c;
        if (col >= n_out) continue;
        float v = acc[0][c];
        if (a.act) {
            // gate and up pass through the type of the activations first, as they do when the activation is a kernel of its own
            const float g = to_f32(from_f32<T>(acc[0][c])), u = to_f32(from_f32<T>(acc[1][c]));
            v = (g / (1.0f + expf(-g))) * u;
        }
        ((O*)a.out)[(size_t)dst * a.ldo + col] = from_f32<O>(v);
    }
}

LLME_API int llme_grouped_linear(const LlmeGroupedArgs* args, int x_dtype, int w_dtype, int out_dtype, cudaStream_t stream) {
    const LlmeGroupedArgs& a = *args;
    if (a.pairs <= 0 || a.n <= 0) return 0;
    if (!a.x || !a.w || !a.out || !a.offsets || !a.order) LLME_REFUSE("grouped_linear: null pointer");
    if (a.num_experts <= 0 || a.top_k <= 0 || a.k <= 0 || (a.act && a.n % 2)) LLME_REFUSE("grouped_linear: bad size");
    const int n_out = a.act ? a.n / 2 : a.n;
    const int most = a.num_experts < a.pairs ? a.num_experts : a.pairs;
    int tiles = (a.pairs + GM - 1) / GM + most;
    if (tiles > a.pairs) tiles = a.pairs;
    const dim3 grid((n_out + GN - 1) / GN, tiles);
#define LLME_GL(T, W, O) llme_launch(grouped_linear_kernel<T, W, O>, grid, dim3(256), 0, stream, a)
    if (x_dtype == LLME_F32 && w_dtype == LLME_F32 && out_dtype == LLME_F32) LLME_GL(float, float, float);
    else if (x_dtype == LLME_BF16 && w_dtype == LLME_BF16 && out_dtype == LLME_BF16) LLME_GL(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == LLME_BF16 && w_dtype == LLME_BF16 && out_dtype == LLME_F32) LLME_GL(__nv_bfloat16, __nv_bfloat16, float);
    else LLME_REFUSE("grouped_linear: unsupported dtypes %d / %d / %d", x_dtype, w_dtype, out_dtype);
#undef LLME_GL
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- the weighted sum of a token's pairs
__global__ void moe_combine_kernel(const float* __restrict__ y, long long ldy, const float* __restrict__ weights, const float* __restrict__ base,
                                   float* __restrict__ out, int top_k, int cols, const float* __restrict__ base_gate, long long ld_gate) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float share = base && base_gate ? 1.0f / (1.0f + expf(-base_gate[(size_t)t * ld_gate])) : 1.0f;   // the shared expert's gate
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols; j += gridDim.y * blockDim.x) {
        float v = 0.0f;
        for (int k = 0; k < top_k; ++k) v = fmaf(weights[(size_t)t * top_k + k], y[((size_t)t * top_k + k) * ldy + j], v);
        out[(size_t)t * cols + j] = base ? base[(size_t)t * cols + j] * share + v : v;
    }
}

LLME_API int llme_moe_combine_gated(const float* y, long long ldy, const float* weights, const float* base, float* out, int tokens,
                                    int top_k, int cols, const float* base_gate, long long ld_gate, cudaStream_t stream);

LLME_API int llme_moe_combine(const float* y, long long ldy, const float* weights, const float* base, float* out, int tokens,
                              int top_k, int cols, cudaStream_t stream) {
    return llme_moe_combine_gated(y, ldy, weights, base, out, tokens, top_k, cols, nullptr, 0, stream);
}

// The same with base[t] times sigmoid(base_gate[t * ld_gate]) (base_gate NULL: times one).
LLME_API int llme_moe_combine_gated(const float* y, long long ldy, const float* weights, const float* base, float* out, int tokens,
                                    int top_k, int cols, const float* base_gate, long long ld_gate, cudaStream_t stream) {
    if (tokens <= 0 || cols <= 0) return 0;
    if (!y || !weights || !out || top_k <= 0) LLME_REFUSE("moe_combine: null pointer or no choices");
    const int threads = 128;
    int pieces = (cols + threads - 1) / threads;
    const int wanted = (592 + tokens - 1) / tokens;
    if (pieces > wanted) pieces = wanted;
    llme_launch(moe_combine_kernel, dim3(tokens, pieces < 1 ? 1 : pieces), dim3(threads), 0, stream, y, ldy, weights, base, out, top_k, cols, base_gate, ld_gate);
    LLME_LAUNCH_STATUS();
}

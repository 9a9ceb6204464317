// Memory-bound kernels of the layers that are not the pre-norm transformer body: activations with learned
// coefficients, gates, residual adds that no norm follows, the per-layer token input, and what a latent
// attention does between its down-projection and its cache.  All arithmetic is 32-bit; only storage may be
// bfloat16.  Row strides are free (operands are often column ranges of a wider product), so one launch serves
// every layout.
#include "common.cuh"
#include "kernel_args.h"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

__device__ __forceinline__ float gelu_tanh(float z) {
    const float k = 0.7978845608028654f;                 // sqrt(2 / pi)
    return 0.5f * z * (1.0f + tanhf(k * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ float sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// ----------------------------------------------------------------------------- out = xielu(in)
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ in, long long ld_in, T* __restrict__ out, long long ld_out, int cols,
                             float a_pos, float a_neg) {
    pdl_launch_dependents();
    pdl_wait();
    const T* i = in + (size_t)blockIdx.x * ld_in;
    T* o = out + (size_t)blockIdx.x * ld_out;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols; j += gridDim.y * blockDim.x)
        o[j] = from_f32<T>(xielu(to_f32(i[j]), a_pos, a_neg));
}

// Rows are few and wide in a decode step and many in a prompt: a second grid dimension walks the columns in pieces, as
// many as it takes to put about four blocks on every SM, each thread then handling a handful of values.
static dim3 grid_for(int rows, int cols, int threads) {
    int pieces = (cols + threads - 1) / threads;
    const int wanted = (592 + rows - 1) / rows;
    if (pieces > wanted) pieces = wanted;
    return dim3(rows, pieces < 1 ? 1 : pieces);
}

// bfloat16 rows of whole 16-byte pieces: eight values per thread and load
__global__ void xielu_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in, __nv_bfloat16* __restrict__ out, long long ld_out,
                                    int cols, float a_pos, float a_neg) {
    pdl_launch_dependents();
    pdl_wait();
    const uint4* i = reinterpret_cast<const uint4*>(in + (size_t)blockIdx.x * ld_in);
    uint4* o = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * ld_out);
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols / 8; j += gridDim.y * blockDim.x) {
        uint4 v = i[j];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            h[e] = __floats2bfloat162_rn(xielu_bf16(f.x, a_pos, a_neg), xielu_bf16(f.y, a_pos, a_neg));
        }
        o[j] = v;
    }
}

LLME_API int llme_xielu(const void* in, long long ld_in, void* out, long long ld_out, int dtype, int rows, int cols,
                        float a_pos, float a_neg, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!in || !out) LLME_REFUSE("xielu: null pointer");
    const int threads = 128;
    if (dtype == LLME_BF16 && cols % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        llme_launch(xielu_bf16x8_kernel, grid_for(rows, cols / 8, threads), dim3(threads), 0, stream, (const __nv_bfloat16*)in, ld_in,
                    (__nv_bfloat16*)out, ld_out, cols, a_pos, a_neg);
        LLME_LAUNCH_STATUS();
    }
    if (dtype == LLME_F32) llme_launch(xielu_kernel<float>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const float*)in, ld_in, (float*)out, ld_out, cols, a_pos, a_neg);
    else if (dtype == LLME_BF16) llme_launch(xielu_kernel<__nv_bfloat16>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const __nv_bfloat16*)in, ld_in, (__nv_bfloat16*)out, ld_out, cols, a_pos, a_neg);
    else LLME_REFUSE("xielu: unsupported dtype %d", dtype);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- out = a * sigmoid(b) * scale
// `group` > 1: b has one value for every `group` neighbouring columns of a (one gate per head).
template <typename T>
__global__ void sigmoid_mul_kernel(const T* __restrict__ a, long long lda, const T* __restrict__ b, long long ldb, T* __restrict__ out,
                                   long long ldo, int cols, float scale, int group) {
    pdl_launch_dependents();
    pdl_wait();
    const T* ar = a + (size_t)blockIdx.x * lda;
    const T* br = b + (size_t)blockIdx.x * ldb;
    T* o = out + (size_t)blockIdx.x * ldo;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols; j += gridDim.y * blockDim.x)
        o[j] = from_f32<T>((to_f32(ar[j]) * sigmoid(to_f32(br[group > 1 ? j / group : j]))) * scale);
}

LLME_API int llme_sigmoid_mul_grouped(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo, int dtype,
                                      int rows, int cols, float scale, int group, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!a || !b || !out) LLME_REFUSE("sigmoid_mul: null pointer");
    if (group < 1 || cols % group) LLME_REFUSE("sigmoid_mul: %d columns are not whole groups of %d", cols, group);
    const int threads = 128;
    if (dtype == LLME_F32) llme_launch(sigmoid_mul_kernel<float>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const float*)a, lda, (const float*)b, ldb, (float*)out, ldo, cols, scale, group);
    else if (dtype == LLME_BF16) llme_launch(sigmoid_mul_kernel<__nv_bfloat16>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)b, ldb, (__nv_bfloat16*)out, ldo, cols, scale, group);
    else LLME_REFUSE("sigmoid_mul: unsupported dtype %d", dtype);
    LLME_LAUNCH_STATUS();
}

LLME_API int llme_sigmoid_mul_scaled(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo, int dtype,
                                     int rows, int cols, float scale, cudaStream_t stream) {
    return llme_sigmoid_mul_grouped(a, lda, b, ldb, out, ldo, dtype, rows, cols, scale, 1, stream);
}

LLME_API int llme_sigmoid_mul(const void* a, long long lda, const void* b, long long ldb, void* out, long long ldo, int dtype,
                              int rows, int cols, cudaStream_t stream) {
    return llme_sigmoid_mul_scaled(a, lda, b, ldb, out, ldo, dtype, rows, cols, 1.0f, stream);
}

// ----------------------------------------------------------------------------- x += a (+ b), optionally a copy of x in another type
// With `a_scale` / `b_scale` (vectors of the row's width) a contribution is multiplied by its vector first.
template <typename A, typename C>
__global__ void residual_add_kernel(float* __restrict__ x, const A* __restrict__ a, const A* __restrict__ b, C* __restrict__ copy, int cols,
                                    const float* __restrict__ a_scale, const float* __restrict__ b_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * cols;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols; j += gridDim.y * blockDim.x) {
        float v = to_f32(a[base + j]);
        if (a_scale) v *= a_scale[j];
        if (b) v += b_scale ? to_f32(b[base + j]) * b_scale[j] : to_f32(b[base + j]);
        v = x[base + j] + v;                 // the sublayers' contributions are summed first, then added to the stream
        x[base + j] = v;
        if (copy) copy[base + j] = from_f32<C>(v);
    }
}

LLME_API int llme_residual_add_scaled(float* x, const void* a, const void* b, int ab_dtype, void* copy, int copy_dtype, int rows, int cols,
                                      const float* a_scale, const float* b_scale, cudaStream_t stream);

LLME_API int llme_residual_add(float* x, const void* a, const void* b, int ab_dtype, void* copy, int copy_dtype, int rows, int cols,
                               cudaStream_t stream) {
    return llme_residual_add_scaled(x, a, b, ab_dtype, copy, copy_dtype, rows, cols, nullptr, nullptr, stream);
}

LLME_API int llme_residual_add_scaled(float* x, const void* a, const void* b, int ab_dtype, void* copy, int copy_dtype, int rows, int cols,
                                      const float* a_scale, const float* b_scale, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!x || !a) LLME_REFUSE("residual_add: null pointer");
    const int threads = 128;
#define LLME_RA(A, C) llme_launch(residual_add_kernel<A, C>, grid_for(rows, cols, threads), dim3(threads), 0, stream, x, (const A*)a, (const A*)b, (C*)copy, cols, a_scale, b_scale)
    if (ab_dtype == LLME_F32 && (copy_dtype == LLME_F32 || !copy)) LLME_RA(float, float);
    else if (ab_dtype == LLME_F32 && copy_dtype == LLME_BF16) LLME_RA(float, __nv_bfloat16);
    else if (ab_dtype == LLME_BF16 && (copy_dtype == LLME_BF16 || !copy)) LLME_RA(__nv_bfloat16, __nv_bfloat16);
    else if (ab_dtype == LLME_BF16 && copy_dtype == LLME_F32) LLME_RA(__nv_bfloat16, float);
    else LLME_REFUSE("residual_add: unsupported dtypes %d / %d", ab_dtype, copy_dtype);
#undef LLME_RA
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- g = gelu_tanh(z) * table[id][offset + j]
template <typename T, typename W>
__global__ void gelu_gather_mul_kernel(const T* __restrict__ z, long long ldz, const int* __restrict__ ids, const W* __restrict__ table,
                                       long long ld_table, int offset, int vocab, T* __restrict__ out, long long ldo, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const int id = ids[blockIdx.x];
    const bool ok = id >= 0 && id < vocab;
    const W* e = table + (size_t)(ok ? id : 0) * ld_table + offset;
    const T* zr = z + (size_t)blockIdx.x * ldz;
    T* o = out + (size_t)blockIdx.x * ldo;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols; j += gridDim.y * blockDim.x)
        o[j] = from_f32<T>(ok ? gelu_tanh(to_f32(zr[j])) * to_f32(e[j]) : 0.0f);
}

LLME_API int llme_gelu_gather_mul(const void* z, long long ldz, int dtype, const int* ids, const void* table, int table_dtype,
                                  long long ld_table, int offset, int vocab, void* out, long long ldo, int rows, int cols,
                                  cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!z || !ids || !table || !out) LLME_REFUSE("gelu_gather_mul: null pointer");
    if (table_dtype != dtype) LLME_REFUSE("gelu_gather_mul: the table is stored in the type of the activations");
    const int threads = cols >= 256 ? 256 : (cols >= 64 ? 64 : 32);
    if (dtype == LLME_F32) llme_launch(gelu_gather_mul_kernel<float, float>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const float*)z, ldz, ids, (const float*)table, ld_table, offset, vocab, (float*)out, ldo, cols);
    else if (dtype == LLME_BF16) llme_launch(gelu_gather_mul_kernel<__nv_bfloat16, __nv_bfloat16>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const __nv_bfloat16*)z, ldz, ids, (const __nv_bfloat16*)table, ld_table, offset, vocab, (__nv_bfloat16*)out, ldo, cols);
    else LLME_REFUSE("gelu_gather_mul: unsupported dtype %d", dtype);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- x += y / sqrt(mean(y^2) + eps) * gain
template <typename G>
__global__ void rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const G* __restrict__ gain, int cols, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * cols;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        const float v = y[base + j];
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)cols + eps);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) x[base + j] += (y[base + j] * rinv) * to_f32(gain[j]);
}

LLME_API int llme_rmsnorm_add(float* x, const float* y, const void* gain, int gain_dtype, int rows, int cols, float eps,
                              cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!x || !y || !gain) LLME_REFUSE("rmsnorm_add: null pointer");
    const int threads = cols >= 4096 ? 1024 : (cols >= 2048 ? 512 : (cols >= 1024 ? 256 : 128));
    if (gain_dtype == LLME_F32) llme_launch(rmsnorm_add_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, y, (const float*)gain, cols, eps);
    else if (gain_dtype == LLME_BF16) llme_launch(rmsnorm_add_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, y, (const __nv_bfloat16*)gain, cols, eps);
    else LLME_REFUSE("rmsnorm_add: unsupported gain dtype %d", gain_dtype);
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- latent: norm, rotation, cache write
// One value of a vector whose first `dims` coordinates are rotated in rotate-half pairs (i, i + dims/2) by the angle
// position * inv_freq[i], formed in 32-bit; coordinates from `dims` on pass unchanged.
// `interleaved`: the pairs are (2i, 2i + 1) instead.
template <typename T>
__device__ __forceinline__ float rotated_value(const T* __restrict__ v, int idx, int dims, const float* __restrict__ inv_freq, int position,
                                               int interleaved = 0) {
    if (idx >= dims) return to_f32(v[idx]);
    const int half = dims >> 1, i = interleaved ? idx >> 1 : (idx < half ? idx : idx - half);
    const float angle = (float)position * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    const float u = to_f32(v[interleaved ? 2 * i : i]), w = to_f32(v[interleaved ? 2 * i + 1 : i + half]);
    const bool first = interleaved ? !(idx & 1) : idx < half;
    return first ? u * c - w * s : w * c + u * s;
}

template <typename T, typename G>
__global__ void latent_post_kernel(LlmeLatentPostArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x, rank = a.rank, rot = a.rot, width = rank + rot;
    const T* kv = (const T*)a.kv_in + (size_t)t * a.kv_stride;
    const int slot = a.slot_mapping ? a.slot_mapping[t] : -1;
    const int pos = a.positions[t];
    T* row = (a.cache && slot >= 0) ? (T*)a.cache + (size_t)slot * width : nullptr;
    if (row && blockIdx.y == 0) {                       // uniform over the block
        float ss = 0.0f;
        for (int j = threadIdx.x; j < rank; j += blockDim.x) {
            const float v = to_f32(kv[j]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float rinv = 1.0f / sqrtf(ss / (float)rank + a.eps);
        const G* gain = (const G*)a.c_gain;
        for (int j = threadIdx.x; j < rank; j += blockDim.x) row[j] = from_f32<T>((to_f32(kv[j]) * rinv) * to_f32(gain[j]));
        for (int j = threadIdx.x; j < rot; j += blockDim.x) row[rank + j] = from_f32<T>(rotated_value(kv + rank, j, a.rot_dims, a.inv_freq, pos, a.interleaved));
    }
    if (rot > 0 && a.q_rot && a.q && (gridDim.y == 1 || blockIdx.y > 0)) {
        const T* qr = (const T*)a.q_rot + (size_t)t * a.q_rot_stride;
        T* q = (T*)a.q + (size_t)t * a.nh * width;
        const int first = gridDim.y == 1 ? 0 : blockIdx.y - 1, stride = gridDim.y == 1 ? 1 : gridDim.y - 1;
        for (int e = first * blockDim.x + threadIdx.x; e < a.nh * rot; e += stride * blockDim.x) {
            const int h = e / rot, j = e - h * rot;
            q[(size_t)h * width + rank + j] = from_f32<T>(rotated_value(qr + (size_t)h * a.q_rot_head_stride, j, a.rot_dims, a.inv_freq, pos, a.interleaved));
        }
    }
}

LLME_API int llme_latent_post(const LlmeLatentPostArgs* args, int dtype, cudaStream_t stream) {
    const LlmeLatentPostArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (!a.kv_in || !a.c_gain || !a.positions) LLME_REFUSE("latent_post: null pointer");
    if (a.rank <= 0 || a.rot < 0 || a.nh <= 0) LLME_REFUSE("latent_post: non-positive size");
    if (a.rot > 0 && (!a.inv_freq || a.rot_dims <= 0 || a.rot_dims % 2 || a.rot_dims > a.rot))
        LLME_REFUSE("latent_post: %d rotated coordinates of %d need frequencies and an even count", a.rot_dims, a.rot);
    const int threads = 128;
    // block (t, 0) norms, rotates and stores the token's cache row; blocks (t, 1..) rotate the heads' query parts
    int q_blocks = a.rot > 0 && a.q_rot ? (a.nh * a.rot + threads - 1) / threads : 0;
    if (q_blocks > 8) q_blocks = 8;
    if (a.tokens > 256) q_blocks = q_blocks ? 1 : 0;
    const dim3 grid(a.tokens, 1 + q_blocks);
#define LLME_LP(T, G) llme_launch(latent_post_kernel<T, G>, grid, dim3(threads), 0, stream, a)
    if (dtype == LLME_F32 && a.gain_dtype == LLME_F32) LLME_LP(float, float);
    else if (dtype == LLME_BF16 && a.gain_dtype == LLME_BF16) LLME_LP(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == LLME_BF16 && a.gain_dtype == LLME_F32) LLME_LP(__nv_bfloat16, float);
    else LLME_REFUSE("latent_post: unsupported dtypes %d / %d", dtype, a.gain_dtype);
#undef LLME_LP
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- out = x / sqrt(mean(x^2) + eps) * gain over strided rows
// A norm on (a column range of) a product: one warp per row for rows of up to 1,024 values, a block per row beyond that.
template <typename X, typename G, typename O>
__global__ void row_norm_kernel(const X* __restrict__ x, long long ldx, const G* __restrict__ gain, O* __restrict__ out, long long ldo,
                                int rows, int cols, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const bool by_warp = cols <= 1024;
    const int lane = threadIdx.x & 31;
    const long long r = by_warp ? (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
    if (r >= rows) return;                               // (uniform over a warp, and over the block where a block has one row)
    const X* xr = x + (size_t)r * ldx;
    O* o = out + (size_t)r * ldo;
    const int first = by_warp ? lane : threadIdx.x, step = by_warp ? 32 : blockDim.x;
    float ss = 0.0f;
    for (int j = first; j < cols; j += step) {
        const float v = to_f32(xr[j]);
        ss += v * v;
    }
    ss = by_warp ? warp_sum(ss) : block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)cols + eps);
    for (int j = first; j < cols; j += step) o[j] = from_f32<O>((to_f32(xr[j]) * rinv) * to_f32(gain[j]));
}

LLME_API int llme_row_norm(const void* x, long long ldx, int x_dtype, const void* gain, int gain_dtype, void* out, long long ldo, int out_dtype,
                           int rows, int cols, float eps, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!x || !gain || !out) LLME_REFUSE("row_norm: null pointer");
    if (!(eps > 0.0f)) LLME_REFUSE("row_norm: eps must be positive");
    const bool by_warp = cols <= 1024;
    const dim3 grid(by_warp ? (rows + 3) / 4 : rows), block(by_warp ? 128 : 256);
#define LLME_RN(X, G, O) llme_launch(row_norm_kernel<X, G, O>, grid, block, 0, stream, (const X*)x, ldx, (const G*)gain, (O*)out, ldo, rows, cols, eps)
    typedef __nv_bfloat16 bf;
    if (x_dtype == LLME_F32 && gain_dtype == LLME_F32 && out_dtype == LLME_F32) LLME_RN(float, float, float);
    else if (x_dtype == LLME_BF16 && gain_dtype == LLME_BF16 && out_dtype == LLME_BF16) LLME_RN(bf, bf, bf);
    else if (x_dtype == LLME_BF16 && gain_dtype == LLME_F32 && out_dtype == LLME_BF16) LLME_RN(bf, float, bf);
    else if (x_dtype == LLME_F32 && gain_dtype == LLME_F32 && out_dtype == LLME_BF16) LLME_RN(float, float, bf);
    else if (x_dtype == LLME_F32 && gain_dtype == LLME_BF16 && out_dtype == LLME_BF16) LLME_RN(float, bf, bf);
    else LLME_REFUSE("row_norm: unsupported dtypes %d / %d / %d", x_dtype, gain_dtype, out_dtype);
#undef LLME_RN
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- the norm on a sublayer's output
// accumulate: x += y / sqrt(mean(y^2) + eps) * gain; else x = ... (y may be x itself: a value is read and written by
// the same thread, after the sum of squares is complete).  Without y nothing is added.  `copy`, if given, receives the
// new x in its own type: the next sublayer's products read it.
template <typename Y, typename G, typename C>
__global__ void postnorm_kernel(float* x, const Y* y, const G* __restrict__ gain, C* __restrict__ copy, int cols, float eps,
                                int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * cols;
    float rinv = 0.0f;
    if (y) {
        float ss = 0.0f;
        for (int j = threadIdx.x; j < cols; j += blockDim.x) {
            const float v = to_f32(y[base + j]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        rinv = 1.0f / sqrtf(ss / (float)cols + eps);
    }
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        float v = accumulate || !y ? x[base + j] : 0.0f;
        if (y) {
            v += (to_f32(y[base + j]) * rinv) * to_f32(gain[j]);
            x[base + j] = v;
        }
        if (copy) copy[base + j] = from_f32<C>(v);
    }
}

// The same for 32-bit y in rows of whole 16-byte pieces: a row is read once and stays in registers between the sum of
// squares and the update, 16 bytes a load.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<const unsigned*>(&lo);
    v.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

template <typename G, typename C, int V>
__global__ void postnorm_vec_kernel(float* x, const float* y, const G* __restrict__ gain, C* __restrict__ copy, int cols, float eps,
                                    int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * cols;
    const int n4 = cols >> 2;
    float4 v[V];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        v[i] = idx < n4 ? reinterpret_cast<const float4*>(y + base)[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)cols + eps);
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx >= n4) continue;
        float4 o = accumulate ? reinterpret_cast<const float4*>(x + base)[idx] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const G* g = gain + 4 * idx;
        o.x += (v[i].x * rinv) * to_f32(g[0]);
        o.y += (v[i].y * rinv) * to_f32(g[1]);
        o.z += (v[i].z * rinv) * to_f32(g[2]);
        o.w += (v[i].w * rinv) * to_f32(g[3]);
        reinterpret_cast<float4*>(x + base)[idx] = o;
        if (copy) store4(copy + base + 4 * idx, o.x, o.y, o.z, o.w);
    }
}

template <typename G, typename C>
static void launch_postnorm_vec(float* x, const float* y, const void* gain, void* copy, int rows, int cols, float eps, int accumulate,
                                cudaStream_t stream) {
    const int n4 = cols / 4;
    int threads = n4 < 1024 ? ((n4 + 31) / 32) * 32 : 1024;
    if (n4 > 1024 && n4 <= 2048) threads = ((n4 / 2 + 31) / 32) * 32;
    const int per = (n4 + threads - 1) / threads;
    if (per <= 1) llme_launch(postnorm_vec_kernel<G, C, 1>, dim3(rows), dim3(threads), 0, stream, x, y, (const G*)gain, (C*)copy, cols, eps, accumulate);
    else if (per <= 2) llme_launch(postnorm_vec_kernel<G, C, 2>, dim3(rows), dim3(threads), 0, stream, x, y, (const G*)gain, (C*)copy, cols, eps, accumulate);
    else llme_launch(postnorm_vec_kernel<G, C, 4>, dim3(rows), dim3(threads), 0, stream, x, y, (const G*)gain, (C*)copy, cols, eps, accumulate);
}

LLME_API int llme_postnorm(float* x, const void* y, int y_dtype, const void* gain, int gain_dtype, void* copy, int copy_dtype,
                           int rows, int cols, float eps, int accumulate, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!x || (y && !gain) || (!y && !copy)) LLME_REFUSE("postnorm: null pointer");
    if (y && !(eps > 0.0f)) LLME_REFUSE("postnorm: eps must be positive");
    if (copy && copy_dtype != LLME_BF16 && copy_dtype != LLME_F32) LLME_REFUSE("postnorm: unsupported copy dtype %d", copy_dtype);
    if (y && y_dtype == LLME_F32 && cols % 4 == 0 && cols <= 16384 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)copy) & 15) == 0 &&
        (gain_dtype == LLME_F32 || gain_dtype == LLME_BF16)) {
        const bool c32 = copy && copy_dtype == LLME_F32;
        if (gain_dtype == LLME_F32 && c32) launch_postnorm_vec<float, float>(x, (const float*)y, gain, copy, rows, cols, eps, accumulate, stream);
        else if (gain_dtype == LLME_F32) launch_postnorm_vec<float, __nv_bfloat16>(x, (const float*)y, gain, copy, rows, cols, eps, accumulate, stream);
        else if (c32) launch_postnorm_vec<__nv_bfloat16, float>(x, (const float*)y, gain, copy, rows, cols, eps, accumulate, stream);
        else launch_postnorm_vec<__nv_bfloat16, __nv_bfloat16>(x, (const float*)y, gain, copy, rows, cols, eps, accumulate, stream);
        LLME_LAUNCH_STATUS();
    }
    const int threads = cols >= 4096 ? 1024 : (cols >= 2048 ? 512 : (cols >= 1024 ? 256 : 128));
#define LLME_PN(Y, G, C) llme_launch(postnorm_kernel<Y, G, C>, dim3(rows), dim3(threads), 0, stream, x, (const Y*)y, (const G*)gain, (C*)copy, cols, eps, accumulate)
#define LLME_PN_C(Y, G) do { if (copy && copy_dtype == LLME_F32) LLME_PN(Y, G, float); else LLME_PN(Y, G, __nv_bfloat16); } while (0)
    if (!y) LLME_PN_C(float, float);
    else if (y_dtype == LLME_F32 && gain_dtype == LLME_F32) LLME_PN_C(float, float);
    else if (y_dtype == LLME_F32 && gain_dtype == LLME_BF16) LLME_PN_C(float, __nv_bfloat16);
    else if (y_dtype == LLME_BF16 && gain_dtype == LLME_F32) LLME_PN_C(__nv_bfloat16, float);
    else if (y_dtype == LLME_BF16 && gain_dtype == LLME_BF16) LLME_PN_C(__nv_bfloat16, __nv_bfloat16);
    else LLME_REFUSE("postnorm: unsupported dtypes %d / %d", y_dtype, gain_dtype);
#undef LLME_PN_C
#undef LLME_PN
    LLME_LAUNCH_STATUS();
}

// ----------------------------------------------------------------------------- out = act(gate, up), gate_up = [gate | up] by columns
// act 0: g sigmoid(g) u.  act 2: gelu(g) u, the tanh form.  act 1 (p0 = limit, p1 = slope): g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(slope g') (u' + 1).
__device__ __forceinline__ float gated_activation(int act, float g, float u, float p0, float p1) {
    if (act == 1) {
        g = fminf(g, p0);
        u = fminf(fmaxf(u, -p0), p0);
        return (g * sigmoid(p1 * g)) * (u + 1.0f);
    }
    if (act == 2) return gelu_tanh(g) * u;
    return (g * sigmoid(g)) * u;
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, long long ld_in, T* __restrict__ out, long long ld_out, int cols, int act, float p0,
                                 float p1, const float* __restrict__ bias) {
    pdl_launch_dependents();
    pdl_wait();
    const T* i = gate_up + (size_t)blockIdx.x * ld_in;
    T* o = out + (size_t)blockIdx.x * ld_out;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols; j += gridDim.y * blockDim.x) {
        float g = to_f32(i[j]), u = to_f32(i[cols + j]);
        if (bias) {                       // the projections' biases [gate | up], added before the activation; each sum
            g = to_f32(from_f32<T>(g + bias[j]));          // is a projection's output and takes its type
            u = to_f32(from_f32<T>(u + bias[cols + j]));
        }
        o[j] = from_f32<T>(gated_activation(act, g, u, p0, p1));
    }
}

LLME_API int llme_gated_act_bias(const void* gate_up, long long ld_in, void* out, long long ld_out, int dtype, int rows, int cols, int act,
                                 float p0, float p1, const float* bias, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!gate_up || !out) LLME_REFUSE("gated_act: null pointer");
    if (act < 0 || act > 2) LLME_REFUSE("gated_act: unknown activation %d", act);
    const int threads = 128;
    if (dtype == LLME_F32) llme_launch(gated_act_kernel<float>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const float*)gate_up, ld_in, (float*)out, ld_out, cols, act, p0, p1, bias);
    else if (dtype == LLME_BF16) llme_launch(gated_act_kernel<__nv_bfloat16>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up, ld_in, (__nv_bfloat16*)out, ld_out, cols, act, p0, p1, bias);
    else LLME_REFUSE("gated_act: unsupported dtype %d", dtype);
    LLME_LAUNCH_STATUS();
}

LLME_API int llme_gated_act(const void* gate_up, long long ld_in, void* out, long long ld_out, int dtype, int rows, int cols, int act,
                            float p0, float p1, cudaStream_t stream) {
    return llme_gated_act_bias(gate_up, ld_in, out, ld_out, dtype, rows, cols, act, p0, p1, nullptr, stream);
}

// ----------------------------------------------------------------------------- out[r, :] += bias: a projection's bias behind a product without one
template <typename T>
__global__ void bias_add_kernel(T* __restrict__ out, long long ld, const float* __restrict__ bias, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    T* o = out + (size_t)blockIdx.x * ld;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < cols; j += gridDim.y * blockDim.x) o[j] = from_f32<T>(to_f32(o[j]) + bias[j]);
}

LLME_API int llme_bias_add(void* out, long long ld, int dtype, const float* bias, int rows, int cols, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (!out || !bias) LLME_REFUSE("bias_add: null pointer");
    const int threads = 128;
    if (dtype == LLME_F32) llme_launch(bias_add_kernel<float>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (float*)out, ld, bias, cols);
    else if (dtype == LLME_BF16) llme_launch(bias_add_kernel<__nv_bfloat16>, grid_for(rows, cols, threads), dim3(threads), 0, stream, (__nv_bfloat16*)out, ld, bias, cols);
    else LLME_REFUSE("bias_add: unsupported dtype %d", dtype);
    LLME_LAUNCH_STATUS();
}

// Attention over a paged cache of latent rows: per token ONE row [c (rank) | rotated key part (rot)] that all heads
// share.  A head's query has already been carried into the latent space, so its score against a token is the dot
// product with that row, and its output is the weighted sum of the rows' first `rank` values.  An optional sink per
// head joins the softmax denominator with exp(sink_h): the running maximum starts at sink_h and the running sum at
// one, with no value behind it.  With a window W a query sees only the last W keys, its own included; pages the window
// has passed are never read.
//
// The plain kernel below visits keys one at a time, one warp per (token, head), for any sizes and both types; it is
// the whole latent attention of the 32-bit path and the twin that the faster kernels are checked against.
#include "common.cuh"
#include "kernel_args.h"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

template <typename T, int REGS>
__global__ void latent_attention_plain_kernel(LlmeLatentAttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int h = blockIdx.y;
    if (t >= a.tokens) return;
    const int rank = a.rank, width = a.rank + a.rot, ps = a.page_size;
    const int p = a.positions[t];
    const int* bt = a.block_tables + (size_t)a.token_request[t] * a.max_blocks;
    float q[REGS], acc[REGS];
    const T* qp = (const T*)a.q + ((size_t)t * a.nh + h) * width;
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int d = lane + 32 * i;
        q[i] = d < width ? to_f32(qp[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = a.sink ? a.sink[h] : -INFINITY, l = a.sink ? 1.0f : 0.0f;
    const int lo = (a.window > 0 && p - a.window + 1 > 0) ? p - a.window + 1 : 0;     // the first key the window reaches
    for (int j = lo; j <= p; ++j) {
        const int page = bt[j / ps];
        const T* row = (const T*)a.cache + ((size_t)page * ps + (j - (j / ps) * ps)) * width;
        float s = 0.0f, v[REGS];
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int d = lane + 32 * i;
            v[i] = d < width ? to_f32(row[d]) : 0.0f;
            s += q[i] * v[i];
        }
        s = warp_sum(s) * a.scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < REGS; ++i) acc[i] = acc[i] * corr + e * v[i];
        m = m_new;
    }
    T* op = (T*)a.out + ((size_t)t * a.nh + h) * rank;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) op[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
static int launch_plain(const LlmeLatentAttnArgs& a, cudaStream_t s) {
    const int wpb = 4;
    dim3 grid((a.tokens + wpb - 1) / wpb, a.nh);
    const int regs = (a.rank + a.rot + 31) / 32;
#define LLME_LA(R) llme_launch(latent_attention_plain_kernel<T, R>, dim3(grid), dim3(wpb * 32), 0, s, a)
    if (regs <= 2) LLME_LA(2);
    else if (regs <= 4) LLME_LA(4);
    else if (regs <= 6) LLME_LA(6);
    else if (regs <= 10) LLME_LA(10);
    else if (regs <= 18) LLME_LA(18);
    else if (regs <= 36) LLME_LA(36);
    else LLME_REFUSE("latent attention: rows of %d values are wider than 1152", a.rank + a.rot);
#undef LLME_LA
    LLME_LAUNCH_STATUS();
}

LLME_API int llme_latent_attention_plain(const LlmeLatentAttnArgs* args, int dtype, cudaStream_t stream) {
    const LlmeLatentAttnArgs& a = *args;
    if (a.tokens <= 0) return 0;
    if (!a.q || !a.cache || !a.out || !a.positions || !a.token_request || !a.block_tables) LLME_REFUSE("latent attention: null pointer");
    if (a.nh <= 0 || a.rank <= 0 || a.rot < 0 || a.page_size <= 0 || a.max_blocks <= 0 || a.window < 0) LLME_REFUSE("latent attention: non-positive size");
    if (a.nh > 65535) LLME_REFUSE("latent attention: more than 65535 heads");
    if (dtype == LLME_F32) return launch_plain<float>(a, stream);
    if (dtype == LLME_BF16) return launch_plain<__nv_bfloat16>(a, stream);
    LLME_REFUSE("latent attention: unsupported dtype %d", dtype);
}

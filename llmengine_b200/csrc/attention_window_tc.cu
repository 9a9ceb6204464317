// Window attention with a sink on the tensor cores (bfloat16, mma.sync m16n8k16, 32-bit scores and sums), compiled per
// pair of sizes: -DDK=<query/key size> -DDV=<value size>, multiples of 16 up to 128.
//
// A block owns 64 rows of one (request, key/value head): a row is a (token, query head of the group) pair, so the heads
// that share a key/value head share every key tile, and a decoded token is one tile of `group` rows.  Keys are walked in
// chunks of 64 positions through a two-stage cp.async pipeline, row by row through the block table: first the chunks
// that hold the request's kept first positions, then the chunks of the window.  A row of a chunk that no query of the
// tile can see is zero-filled and never read, so a page that was given back is never touched.  Each of the four warps
// owns 16 rows: S = Q K^T with the queries kept in registers, the mask (j <= i and (i - j < window or j < keep_first)),
// an optional cap on the scores (s <- c tanh(s / c)), an online softmax whose running maximum starts at the sink and whose sum starts at one (the sink's own term), and
// O += P V with the probabilities taken straight from the score registers.
//
// Single decoded tokens: a request's chunks are dealt out to `splits` blocks (a window of a thousand keys is seventeen
// chunks, and eight requests of four key/value heads alone would leave most of the GPU idle); each writes its running
// maximum, sum and unnormalised output per row to scratch memory, and a second kernel adds the parts and the sink.
#include "common.cuh"
#include "kernel_args.h"

#ifndef DK
#error "compile with -DDK=<query/key size> -DDV=<value size>"
#endif
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK >= 16 && DV >= 16 && DK <= 128 && DV <= 128, "sizes: multiples of 16 up to 128");

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BM = 64, BN = 64, THREADS = 128;
constexpr int LDK = DK + 8, LDV = DV + 8;
constexpr int STAGE_ELEMS = BN * LDK + BN * LDV;
constexpr int SMEM_BYTES = 2 * STAGE_ELEMS * (int)sizeof(bf16);
static_assert(BM * LDK <= STAGE_ELEMS, "the query tile is staged in the first key stage");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* d, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const unsigned*>(&v);
}

__global__ void __launch_bounds__(THREADS) window_tc_kernel(LlmeWindowFastArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    pdl_wait();                                           // queries and the newest cache rows come from the kernel before
    const int req = a.rows[blockIdx.z];
    const int q0 = a.cu_q_lens[req], q_len = a.cu_q_lens[req + 1] - q0, ctx = a.ctx_lens[req], start = ctx - q_len;
    const int G = a.nh / a.nkv, total_rows = q_len * G, tile0 = a.splits > 1 ? 0 : blockIdx.x * BM;
    if (tile0 >= total_rows) return;
    const int kvh = blockIdx.y, ps = a.page_size;
    const int last_row = min(total_rows, tile0 + BM) - 1;
    const int p_lo = start + tile0 / G, p_hi = start + last_row / G;
    const int W = a.window;
    const int lo_min = (W > 0 && p_lo - W + 1 > 0) ? p_lo - W + 1 : 0;             // the first key the tile's window reaches
    const int first_eff = a.keep_first < lo_min ? a.keep_first : lo_min;           // keys 0 .. first_eff-1 are seen beside it
    const int cw = lo_min / BN, c_end = p_hi / BN;
    const int nf = min((first_eff + BN - 1) / BN, cw);
    const int n_chunks = nf + (c_end - cw + 1);
    // with splits, blockIdx.x is not a row tile (there is one) but a share of the chunks
    const bool split = a.splits > 1;
    if (split) pdl_launch_dependents();                   // the few blocks of the kernel that adds the parts may move in
    const int per = split ? (n_chunks + a.splits - 1) / a.splits : n_chunks;
    const int c_first = split ? min(n_chunks, (int)blockIdx.x * per) : 0;
    const int c_stop = split ? min(n_chunks, c_first + per) : n_chunks;
    const int* bt = a.block_tables + (size_t)a.table_rows[req] * a.max_blocks;
    const size_t page_elems = (size_t)a.nkv * ps * (DK + DV);
    const bf16* cache = (const bf16*)a.cache;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Eight threads bring one row (its page is looked up once, 128 bytes of it go in one request), sixteen rows a pass.
    const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
    auto load_chunk = [&](int stage, int chunk) {
        bf16* Ks = smem + stage * STAGE_ELEMS;
        bf16* Vs = Ks + BN * LDK;
        const int j0 = chunk * BN;
        constexpr int KC = DK / 8, VC = DV / 8, TPR = 8;
        const int c0 = threadIdx.x % TPR;
        for (int r = threadIdx.x / TPR; r < BN; r += THREADS / TPR) {
            const int j = j0 + r;
            const bool needed = j <= p_hi && (j >= lo_min || j < first_eff);
            const int blk = ps_shift >= 0 ? j >> ps_shift : j / ps;
            const int page = needed ? bt[blk] : -1;
            const bool ok = page >= 0;
            const int off = j - blk * ps;
            const bf16* krow = ok ? cache + (size_t)page * page_elems + ((size_t)kvh * ps + off) * DK : cache;
            const bf16* vrow = ok ? cache + (size_t)page * page_elems + (size_t)a.nkv * ps * DK + ((size_t)kvh * ps + off) * DV : cache;
#pragma unroll
            for (int c = c0; c < KC; c += TPR) cp_async16(Ks + r * LDK + c * 8, ok ? krow + c * 8 : cache, ok);
#pragma unroll
            for (int c = c0; c < VC; c += TPR) cp_async16(Vs + r * LDV + c * 8, ok ? vrow + c * 8 : cache, ok);
        }
        cp_async_commit();
    };

    // the queries: through the first key stage into registers
    {
        const bf16* q = (const bf16*)a.q;
        for (int i = threadIdx.x; i < BM * (DK / 8); i += THREADS) {
            const int r = i / (DK / 8), c = i % (DK / 8);
            const int row = tile0 + r;
            const bool ok = row < total_rows;
            const size_t token = q0 + (ok ? row / G : 0);
            const int head = kvh * G + (ok ? row % G : 0);
            cp_async16(smem + r * LDK + c * 8, q + (token * a.nh + head) * DK + c * 8, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
    }
    unsigned qf[DK / 16][4];
#pragma unroll
    for (int k = 0; k < DK / 16; ++k)
        ldmatrix_x4(qf[k][0], qf[k][1], qf[k][2], qf[k][3], smem + (warp * 16 + (lane & 15)) * LDK + k * 16 + (lane >> 4) * 8);
    __syncthreads();

    // this thread's two rows: r0 = lane / 4 and r0 + 8 of the warp's 16
    int pos[2];
    bool valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = tile0 + warp * 16 + (lane >> 2) + h * 8;
        valid[h] = row < total_rows;
        pos[h] = start + (valid[h] ? row / G : 0);
    }
    const float LOG2E = 1.4426950408889634f;
    const float cap = a.softcap, cap2 = cap * LOG2E;      // with a cap c: s <- c tanh(scale s / c), then to base 2
    const float sc = cap > 0.0f ? a.scale / cap : a.scale * LOG2E;
    float m[2], l[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = tile0 + warp * 16 + (lane >> 2) + h * 8;
        const int head = kvh * G + (valid[h] ? row % G : 0);
        const bool with_sink = a.sink && !split;          // (with splits the second kernel adds it)
        m[h] = with_sink ? a.sink[head] * LOG2E : -INFINITY;  // the sink: a score that is not scaled and has no value
        l[h] = with_sink ? 1.0f : 0.0f;
    }
    float o[DV / 8][4];
#pragma unroll
    for (int n = 0; n < DV / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.0f;

    auto chunk_at = [&](int i) { return i < nf ? i : cw + (i - nf); };
    if (c_first < c_stop) load_chunk(c_first & 1, chunk_at(c_first));
    for (int ci = c_first; ci < c_stop; ++ci) {
        if (ci + 1 < c_stop) {
            load_chunk((ci + 1) & 1, chunk_at(ci + 1));
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* Ks = smem + (ci & 1) * STAGE_ELEMS;
        const bf16* Vs = Ks + BN * LDK;
        const int j0 = chunk_at(ci) * BN;

        float s[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[n][i] = 0.0f;
#pragma unroll
        for (int k = 0; k < DK / 16; ++k)
#pragma unroll
            for (int n = 0; n < BN / 8; n += 2) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, Ks + (n * 8 + (lane & 7) + (lane >> 4) * 8) * LDK + k * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[n], qf[k], b0, b1);
                mma_bf16(s[n + 1], qf[k], b2, b3);
            }

        // scale, mask, running maximum; a chunk that every row of the tile sees whole needs no mask
        const bool whole = last_row == tile0 + BM - 1 && j0 + BN - 1 <= p_lo && (W <= 0 || p_hi - j0 < W || j0 + BN <= a.keep_first);
        float mx[2] = {-INFINITY, -INFINITY};
        if (whole) {
#pragma unroll
            for (int n = 0; n < BN / 8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[n][i] = cap > 0.0f ? cap2 * tanhf(s[n][i] * sc) : s[n][i] * sc;
                    mx[i >> 1] = fmaxf(mx[i >> 1], s[n][i]);
                }
        } else {
#pragma unroll
            for (int n = 0; n < BN / 8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int h = i >> 1;
                    const int j = j0 + n * 8 + (lane & 3) * 2 + (i & 1);
                    const bool see = valid[h] && j <= pos[h] && (W <= 0 || pos[h] - j < W || j < a.keep_first);
                    const float v = see ? (cap > 0.0f ? cap2 * tanhf(s[n][i] * sc) : s[n][i] * sc) : -INFINITY;
                    s[n][i] = v;
                    mx[h] = fmaxf(mx[h], v);
                }
        }
        float corr[2], base[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m[h], mx[h]);
            base[h] = m_new == -INFINITY ? 0.0f : m_new;      // a row that has seen nothing yet
            corr[h] = exp2f(m[h] - base[h]);                   // exp2(-inf) = 0
            m[h] = m_new;
        }
        float sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int n = 0; n < BN / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p = exp2f(s[n][i] - base[i >> 1]);
                s[n][i] = p;
                sum[i >> 1] += p;
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
            sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
            l[h] = l[h] * corr[h] + sum[h];
        }
#pragma unroll
        for (int n = 0; n < DV / 8; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
        // O += P V: the probabilities of key tiles 2k and 2k + 1 are the A operand of key step k
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
            unsigned pf[4] = {pack_bf16(s[2 * k][0], s[2 * k][1]), pack_bf16(s[2 * k][2], s[2 * k][3]),
                              pack_bf16(s[2 * k + 1][0], s[2 * k + 1][1]), pack_bf16(s[2 * k + 1][2], s[2 * k + 1][3])};
#pragma unroll
            for (int n = 0; n < DV / 8; n += 2) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, Vs + (k * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + n * 8 + (lane >> 4) * 8);
                mma_bf16(o[n], pf, b0, b1);
                mma_bf16(o[n + 1], pf, b2, b3);
            }
        }
        __syncthreads();
    }

    if (split) {
        // this share's part of every row: maximum, sum, unnormalised output
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (!valid[h]) continue;
            const int row = warp * 16 + (lane >> 2) + h * 8;
            float* part = a.scratch + ((((size_t)blockIdx.z * a.nkv + kvh) * a.splits + blockIdx.x) * G + row) * (DV + 2);
            if ((lane & 3) == 0) {
                part[0] = m[h];
                part[1] = l[h];
            }
#pragma unroll
            for (int n = 0; n < DV / 8; ++n) {
                part[2 + n * 8 + (lane & 3) * 2] = o[n][h * 2];
                part[2 + n * 8 + (lane & 3) * 2 + 1] = o[n][h * 2 + 1];
            }
        }
        return;
    }
    bf16* out = (bf16*)a.out;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!valid[h]) continue;
        const int row = tile0 + warp * 16 + (lane >> 2) + h * 8;
        const size_t token = q0 + row / G;
        const int head = kvh * G + row % G;
        const float inv = 1.0f / l[h];
        bf16* op = out + (token * a.nh + head) * DV + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < DV / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(op + n * 8) = __floats2bfloat162_rn(o[n][h * 2] * inv, o[n][h * 2 + 1] * inv);
    }
}

// One warp per row (a query head of a decoded token): the shares' parts and the sink become the output row.
__global__ void __launch_bounds__(THREADS) window_merge_kernel(LlmeWindowFastArgs a) {
    pdl_wait();                                           // every share has written its part
    const int req = a.rows[blockIdx.y], kvh = blockIdx.x, G = a.nh / a.nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t token = a.cu_q_lens[req];
    const float LOG2E = 1.4426950408889634f;
    for (int row = warp; row < G; row += THREADS / 32) {
        const int head = kvh * G + row;
        const float* parts = a.scratch + (((size_t)blockIdx.y * a.nkv + kvh) * a.splits * G + row) * (DV + 2);
        const size_t stride = (size_t)G * (DV + 2);
        float m = a.sink ? a.sink[head] * LOG2E : -INFINITY;
        for (int s = 0; s < a.splits; ++s) m = fmaxf(m, parts[s * stride]);
        const float base = m == -INFINITY ? 0.0f : m;
        float l = a.sink ? exp2f(a.sink[head] * LOG2E - base) : 0.0f;
        float acc[(DV + 31) / 32];
#pragma unroll
        for (int i = 0; i < (DV + 31) / 32; ++i) acc[i] = 0.0f;
        for (int s = 0; s < a.splits; ++s) {
            const float* p = parts + s * stride;
            const float w = exp2f(p[0] - base);           // a share that saw nothing: exp2(-inf) = 0
            l += p[1] * w;
#pragma unroll
            for (int i = 0; i < (DV + 31) / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < DV) acc[i] += p[2 + d] * w;
            }
        }
        const float inv = 1.0f / l;
        bf16* op = (bf16*)a.out + (token * a.nh + head) * DV;
#pragma unroll
        for (int i = 0; i < (DV + 31) / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < DV) op[d] = __float2bfloat16_rn(acc[i] * inv);
        }
    }
}

}  // namespace

LLME_API long long llme_window_attention_tc_scratch_floats(int n_rows, int nh, int splits) {
    return splits > 1 ? (long long)n_rows * nh * splits * (DV + 2) : 0;
}

LLME_API int llme_window_attention_tc_sizes(int* dk, int* dv) {
    *dk = DK;
    *dv = DV;
    return 0;
}

// The requests `rows` of the batch; `max_q_len` is the longest of their portions (1: single decoded tokens).
LLME_API int llme_window_attention_tc(const LlmeWindowFastArgs* args, int max_q_len, int max_ctx, cudaStream_t stream) {
    const LlmeWindowFastArgs& a = *args;
    (void)max_ctx;
    if (a.n_rows <= 0 || max_q_len <= 0) return 0;
    if (!a.q || !a.cache || !a.out || !a.rows || !a.cu_q_lens || !a.ctx_lens || !a.table_rows || !a.block_tables)
        LLME_REFUSE("window attention: null pointer");
    if (a.nh <= 0 || a.nkv <= 0 || a.nh % a.nkv) LLME_REFUSE("window attention: %d query heads are not a multiple of %d key/value heads", a.nh, a.nkv);
    if (a.page_size <= 0 || a.max_blocks <= 0 || a.window < 0 || a.keep_first < 0) LLME_REFUSE("window attention: bad size");
    if (a.nkv > 65535 || a.n_rows > 65535) LLME_REFUSE("window attention: more than 65535 key/value heads or requests");
    if ((((uintptr_t)a.q | (uintptr_t)a.cache | (uintptr_t)a.out) & 15)) LLME_REFUSE("window attention: operands must be 16-byte aligned");
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(window_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            LLME_REFUSE("window attention: %d bytes of shared memory are not available", SMEM_BYTES);
        configured = true;
    }
    const int G = a.nh / a.nkv;
    const long long tiles = ((long long)max_q_len * G + BM - 1) / BM;
    if (a.splits > 1) {
        if (max_q_len != 1 || G > BM || !a.scratch) LLME_REFUSE("window attention: key ranges are for single tokens of at most %d heads a group, with scratch memory", BM);
        llme_launch(window_tc_kernel, dim3((unsigned)a.splits, a.nkv, a.n_rows), dim3(THREADS), (size_t)SMEM_BYTES, stream, a);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            snprintf(llme_error_buffer(), 512, "%s", cudaGetErrorString(e));
            return (int)e;
        }
        llme_launch(window_merge_kernel, dim3(a.nkv, a.n_rows), dim3(THREADS), 0, stream, a);
        LLME_LAUNCH_STATUS();
    }
    llme_launch(window_tc_kernel, dim3((unsigned)tiles, a.nkv, a.n_rows), dim3(THREADS), (size_t)SMEM_BYTES, stream, a);
    LLME_LAUNCH_STATUS();
}

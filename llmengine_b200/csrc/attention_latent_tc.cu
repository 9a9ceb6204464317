// Tensor-core attention over a paged cache of latent rows [c (RANK) | rotated key part (rot)], bfloat16, compiled per
// latent size (-DRANK=N, a multiple of 64).  All heads of a token read the same rows, so a block's query rows are
// (token, head) pairs of one request and every key tile it loads serves all of them: with H heads a decoded token
// is a tile of H rows, not H separate vectors, and the cache is read once per tile.
//
// A block owns `RG` groups of 16 query rows and walks the keys in tiles of BN.  Per tile its 8 warps
//   1. share the scores: warp (rg, wg) computes S for its 16 rows and its BN/WG keys (mma.sync m16n8k16, Q and the
//      key rows through ldmatrix from shared memory, the full row width rank + rot as the inner dimension),
//   2. agree on every row's maximum through shared memory, turn scores into probabilities and store them as
//      bfloat16 in shared memory,
//   3. share the outputs: warp (rg, wg) adds P V for its 16 rows and its RANK/WG columns, V being the first RANK
//      values of the same key rows (ldmatrix.trans), so nothing is loaded twice.
// Keys arrive through a two-stage cp.async pipeline, page by page through the block table; rows outside the
// needed range are zero-filled, never read.  The running maximum of a row starts at its head's sink (and the
// running sum at one) when the mixer has one.  With a window W a query sees only the last W keys: a tile's walk starts
// at the tile that holds the nearest key any of its rows sees.  A decode step may split the keys of a request over several blocks,
// whose partial sums meet in scratch memory and are merged by a second kernel.
#include "common.cuh"
#include "kernel_args.h"

#ifndef RANK
#error "compile with -DRANK=<latent size>"
#endif
static_assert(RANK % 64 == 0 && RANK >= 64 && RANK <= 1024, "RANK must be a multiple of 64 up to 1024");

LLME_API const char* llme_last_error() { return llme_error_buffer(); }
LLME_API int llme_latent_attention_rank() { return RANK; }

namespace {

constexpr int WARPS = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

struct Args {
    const __nv_bfloat16* q; const __nv_bfloat16* cache; __nv_bfloat16* out;
    const float* sink;
    const int* rows; const int* cu_q_lens; const int* ctx_lens; const int* table_rows; const int* block_tables;
    float* scratch;
    int max_blocks, nh, rot, page_size, splits;
    float scale;
    int window;                                    // W > 0: query i sees key j only if i - j < W
};

// RG groups of 16 query rows, WG = 8 / RG warps per group, key tiles of BN.
template <int RG, int BN, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, RG <= 2 ? 2 : 1) latent_attention_tc_kernel(Args a) {
    constexpr int WG = WARPS / RG, BM = 16 * RG;
    constexpr int KW = BN / WG, NT_S = KW / 8;             // keys and 8-key tiles of a warp's share of the scores
    constexpr int CW = RANK / WG, NT_O = CW / 8;           // columns and 8-column tiles of a warp's share of the outputs
    static_assert(KW % 8 == 0 && CW % 8 == 0, "a warp's share must be whole tiles");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int width = RANK + a.rot, widthp = (width + 63) & ~63, ld = widthp + 8;      // whole groups of four 16-wide steps
    __nv_bfloat16* q_s = (__nv_bfloat16*)smem_raw;                       // [BM][ld]
    __nv_bfloat16* k_s = q_s + (size_t)BM * ld;                          // [2][BN][ld]
    __nv_bfloat16* p_s = k_s + (size_t)STAGES * BN * ld;                 // [BM][BN + 8]
    float* red = (float*)(p_s + (size_t)BM * (BN + 8));                  // [WG][BM]
    constexpr int LDP = BN + 8;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rg = warp % RG, wg = warp / RG;
    const int n = blockIdx.y, split = blockIdx.z;
    const int r = a.rows[n];
    const int tok0 = a.cu_q_lens[r], q_len = a.cu_q_lens[r + 1] - tok0;
    const int H = a.nh, n_rows = q_len * H;
    // the last rows of a prompt see the most keys: their blocks are launched first, so that the long ones do not
    // run alone at the end
    const int row0 = (int)(gridDim.x - 1 - blockIdx.x) * BM;
    if (row0 >= n_rows) return;
    const int ctx = a.ctx_lens[r], first_pos = ctx - q_len;
    const int last_row = min(row0 + BM, n_rows) - 1;
    const int pmax = first_pos + last_row / H;                           // the farthest key any row of the tile sees
    const int W = a.window;
    const int pmin = first_pos + row0 / H;                               // the position of the tile's first row
    const int kmin = (W > 0 && pmin - W + 1 > 0) ? pmin - W + 1 : 0;     // the nearest key any row of the tile sees
    const int tile_lo = kmin / BN, tiles = pmax / BN + 1 - tile_lo;
    // the tiles are dealt out evenly: with more ranges than tiles the later ranges get one tile each or none
    const int t_begin = tile_lo + (int)((long long)split * tiles / a.splits), t_end = tile_lo + (int)((long long)(split + 1) * tiles / a.splits);
    const int* bt = a.block_tables + (size_t)a.table_rows[r] * a.max_blocks;
    const int ps = a.page_size;
    const int chunks = width >> 3;                                       // 16-byte pieces of a row

    // the padding columns of Q and of both key stages are zero for the whole kernel
    if (widthp > width) {
        const int pad = widthp - width;
        for (int e = tid; e < (BM + STAGES * BN) * pad; e += blockDim.x) {
            const int row = e / pad, c = width + e % pad;
            (row < BM ? q_s + (size_t)row * ld : k_s + (size_t)(row - BM) * ld)[c] = __float2bfloat16(0.0f);
        }
    }
    pdl_wait();

    // A warp brings whole key rows: one block-table lookup per row (every lane reads the same entry), the lanes share
    // the row's 16-byte pieces.
    auto load_keys = [&](int tile, int stage) {
        __nv_bfloat16* dst = k_s + (size_t)stage * BN * ld;
        const int j0 = tile * BN;
        for (int kr = warp; kr < BN; kr += WARPS) {
            const int j = j0 + kr;
            __nv_bfloat16* d = dst + (size_t)kr * ld;
            if (j <= pmax && j >= kmin) {                        // (a page the window has passed may be gone: never read)
                const int blk = j / ps;
                const __nv_bfloat16* src = a.cache + ((size_t)bt[blk] * ps + (j - blk * ps)) * width;
                for (int c = lane; c < chunks; c += 32) cp_async16(d + c * 8, src + c * 8);
            } else {
                for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };

    // Q tile: rows (token, head) of one request are contiguous in memory
    {
        const __nv_bfloat16* src = a.q + ((size_t)tok0 * H + row0) * width;
        for (int qr = warp; qr < BM; qr += WARPS) {
            __nv_bfloat16* d = q_s + (size_t)qr * ld;
            if (row0 + qr < n_rows) {
                for (int c = lane; c < chunks; c += 32) cp_async16(d + c * 8, src + (size_t)qr * width + c * 8);
            } else {
                for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(d + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    }
    if (t_begin < t_end) load_keys(t_begin, 0);
    cp_async_commit();
    if (STAGES == 2) {                             // the second tile is requested at once, not when the first has landed
        if (t_begin + 1 < t_end) load_keys(t_begin + 1, 1);
        cp_async_commit();
    }

    // this thread's two rows of its group: lane / 4 and lane / 4 + 8
    const int lr0 = rg * 16 + (lane >> 2), lr1 = lr0 + 8;
    const int gr0 = row0 + lr0, gr1 = row0 + lr1;
    const bool ok0 = gr0 < n_rows, ok1 = gr1 < n_rows;
    const int p0 = ok0 ? first_pos + gr0 / H : -1, p1 = ok1 ? first_pos + gr1 / H : -1;
    const bool with_sink = a.sink != nullptr && split == 0;
    float m0 = (with_sink && ok0) ? a.sink[gr0 % H] : -INFINITY;
    float m1 = (with_sink && ok1) ? a.sink[gr1 % H] : -INFINITY;
    // the sink counts once: in the partial sum of one thread of the row
    float l0 = (with_sink && ok0 && wg == 0 && (lane & 3) == 0) ? 1.0f : 0.0f;
    float l1 = (with_sink && ok1 && wg == 0 && (lane & 3) == 0) ? 1.0f : 0.0f;
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    for (int tile = t_begin; tile < t_end; ++tile) {
        const int stage = STAGES == 1 ? 0 : (tile - t_begin) & 1;
        if (STAGES == 1 && tile > t_begin) {
            __syncthreads();                       // everyone has finished with the tile before this one
            load_keys(tile, 0);
            cp_async_commit();
        }
        if (STAGES == 2) cp_async_wait<1>();       // everything but the newest request: this tile has landed
        else cp_async_wait<0>();
        __syncthreads();
        const __nv_bfloat16* kt = k_s + (size_t)stage * BN * ld;

        // 1. scores of this warp's rows against its share of the tile's keys
        float s[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
        // Four steps of 16 along the row at a time: their fragments are all requested before the first product, so the
        // shared-memory latency of one step hides behind the products of the others (a block is one per SM, eight warps).
        const uint32_t q_addr = smem_u32(q_s + (size_t)(rg * 16 + (lane & 15)) * ld + (lane >> 4) * 8);
        if constexpr (NT_S % 2 == 0) {
            // key fragments of two 8-key tiles per load: matrices (keys 0-7 | 8-15) x (columns 0-7 | 8-15)
            const uint32_t k_addr = smem_u32(kt + (size_t)(wg * KW + (lane & 7) + ((lane >> 4) << 3)) * ld + ((lane >> 3) & 1) * 8);
            for (int ks = 0; ks < widthp / 16; ks += 4) {
                uint32_t qa[4][4], kb[4][NT_S / 2][4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    ldmatrix_x4(q_addr + (ks + u) * 32, qa[u][0], qa[u][1], qa[u][2], qa[u][3]);
#pragma unroll
                    for (int np = 0; np < NT_S / 2; ++np)
                        ldmatrix_x4(k_addr + (uint32_t)(np * 16 * ld * 2) + (ks + u) * 32, kb[u][np][0], kb[u][np][1], kb[u][np][2], kb[u][np][3]);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int np = 0; np < NT_S / 2; ++np) {
                        mma_bf16(s[2 * np], qa[u][0], qa[u][1], qa[u][2], qa[u][3], kb[u][np][0], kb[u][np][1]);
                        mma_bf16(s[2 * np + 1], qa[u][0], qa[u][1], qa[u][2], qa[u][3], kb[u][np][2], kb[u][np][3]);
                    }
            }
        } else {
            const uint32_t k_addr = smem_u32(kt + (size_t)(wg * KW + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
            // one 8-key tile: two accumulators (even and odd steps) keep two products in flight, added at the end
            float s2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int ks = 0; ks < widthp / 16; ks += 4) {
                uint32_t qa[4][4], kb[4][2];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    ldmatrix_x4(q_addr + (ks + u) * 32, qa[u][0], qa[u][1], qa[u][2], qa[u][3]);
                    ldmatrix_x2(k_addr + (ks + u) * 32, kb[u][0], kb[u][1]);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) mma_bf16((u & 1) ? s2 : s[0], qa[u][0], qa[u][1], qa[u][2], qa[u][3], kb[u][0], kb[u][1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) s[0][i] += s2[i];
        }
        // 2. scale, mask, row maxima over the whole tile
        float t0 = -INFINITY, t1 = -INFINITY;
        const int jbase = tile * BN + wg * KW + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
            const int j = jbase + nt * 8;
            s[nt][0] = j <= p0 && (W <= 0 || p0 - j < W) ? s[nt][0] * a.scale : -INFINITY;
            s[nt][1] = j + 1 <= p0 && (W <= 0 || p0 - j - 1 < W) ? s[nt][1] * a.scale : -INFINITY;
            s[nt][2] = j <= p1 && (W <= 0 || p1 - j < W) ? s[nt][2] * a.scale : -INFINITY;
            s[nt][3] = j + 1 <= p1 && (W <= 0 || p1 - j - 1 < W) ? s[nt][3] * a.scale : -INFINITY;
            t0 = fmaxf(t0, fmaxf(s[nt][0], s[nt][1]));
            t1 = fmaxf(t1, fmaxf(s[nt][2], s[nt][3]));
        }
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
        t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
        t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
        if ((lane & 3) == 0) {
            red[wg * BM + lr0] = t0;
            red[wg * BM + lr1] = t1;
        }
        __syncthreads();
        float mn0 = m0, mn1 = m1;
#pragma unroll
        for (int w = 0; w < WG; ++w) {
            mn0 = fmaxf(mn0, red[w * BM + lr0]);
            mn1 = fmaxf(mn1, red[w * BM + lr1]);
        }
        const float ms0 = mn0 == -INFINITY ? 0.0f : mn0, ms1 = mn1 == -INFINITY ? 0.0f : mn1;
        const float c0 = expf(m0 - ms0), c1 = expf(m1 - ms1);            // exp(-inf) = 0 before the first key
        m0 = mn0;
        m1 = mn1;
        float sum0 = 0.0f, sum1 = 0.0f;
        __nv_bfloat16* pr0 = p_s + (size_t)lr0 * LDP + wg * KW + (lane & 3) * 2;
        __nv_bfloat16* pr1 = p_s + (size_t)lr1 * LDP + wg * KW + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < NT_S; ++nt) {
            const float e0 = expf(s[nt][0] - ms0), e1 = expf(s[nt][1] - ms0);
            const float e2 = expf(s[nt][2] - ms1), e3 = expf(s[nt][3] - ms1);
            sum0 += e0 + e1;
            sum1 += e2 + e3;
            *reinterpret_cast<__nv_bfloat162*>(pr0 + nt * 8) = __floats2bfloat162_rn(e0, e1);
            *reinterpret_cast<__nv_bfloat162*>(pr1 + nt * 8) = __floats2bfloat162_rn(e2, e3);
        }
        l0 = l0 * c0 + sum0;
        l1 = l1 * c1 + sum1;
        __syncthreads();
        // 3. outputs: this warp's rows, its share of the columns, all keys of the tile
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
        }
        const uint32_t p_addr = smem_u32(p_s + (size_t)(rg * 16 + (lane & 15)) * LDP + (lane >> 4) * 8);
        // value fragments of two 8-column tiles per load: matrices (keys 0-7 | 8-15) x (columns 0-7 | 8-15), transposed
        const uint32_t v_addr = smem_u32(kt + (size_t)(lane & 15) * ld + wg * CW + (lane >> 4) * 8);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(p_addr + ks * 32, a0, a1, a2, a3);
#pragma unroll
            for (int np = 0; np < NT_O / 2; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(v_addr + (uint32_t)(ks * 16 * ld * 2) + np * 32, b0, b1, b2, b3);
                mma_bf16(o[2 * np], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
            if constexpr (NT_O % 2 == 1) {
                uint32_t b0, b1;
                ldmatrix_x2_trans(v_addr + (uint32_t)(ks * 16 * ld * 2) + (NT_O - 1) * 16, b0, b1);
                mma_bf16(o[NT_O - 1], a0, a1, a2, a3, b0, b1);
            }
        }
        if (STAGES == 2) {                         // the stage is free again: the tile after the next one goes there
            __syncthreads();
            if (tile + 2 < t_end) load_keys(tile + 2, stage);
            cp_async_commit();
        }
    }
    cp_async_wait<0>();

    // row sums: over the four lanes of a row, then over the warps of the group
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();
    if ((lane & 3) == 0) {
        red[wg * BM + lr0] = l0;
        red[wg * BM + lr1] = l1;
    }
    __syncthreads();
    float L0 = 0.0f, L1 = 0.0f;
#pragma unroll
    for (int w = 0; w < WG; ++w) {
        L0 += red[w * BM + lr0];
        L1 += red[w * BM + lr1];
    }
    const int col = wg * CW + (lane & 3) * 2;
    if (a.splits == 1) {
        const float i0 = L0 > 0.0f ? 1.0f / L0 : 0.0f, i1 = L1 > 0.0f ? 1.0f / L1 : 0.0f;
        __nv_bfloat16* out0 = a.out + ((size_t)tok0 * H + gr0) * RANK + col;
        __nv_bfloat16* out1 = a.out + ((size_t)tok0 * H + gr1) * RANK + col;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            if (ok0) *reinterpret_cast<__nv_bfloat162*>(out0 + nt * 8) = __floats2bfloat162_rn(o[nt][0] * i0, o[nt][1] * i0);
            if (ok1) *reinterpret_cast<__nv_bfloat162*>(out1 + nt * 8) = __floats2bfloat162_rn(o[nt][2] * i1, o[nt][3] * i1);
        }
        return;
    }
    // partial sums of this split: [n][split][row][RANK + 2] = unnormalised outputs, maximum, sum
    float* part0 = a.scratch + (((size_t)n * a.splits + split) * n_rows + gr0) * (RANK + 2);
    float* part1 = a.scratch + (((size_t)n * a.splits + split) * n_rows + gr1) * (RANK + 2);
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
        if (ok0) *reinterpret_cast<float2*>(part0 + col + nt * 8) = make_float2(o[nt][0], o[nt][1]);
        if (ok1) *reinterpret_cast<float2*>(part1 + col + nt * 8) = make_float2(o[nt][2], o[nt][3]);
    }
    if (wg == 0 && (lane & 3) == 0) {
        if (ok0) { part0[RANK] = m0; part0[RANK + 1] = L0; }
        if (ok1) { part1[RANK] = m1; part1[RANK + 1] = L1; }
    }
}

// One block per (request of the list, head): the ranges' weights exp(m_s - M) / L are formed once by the first warp,
// then every thread adds its columns over the ranges in their order (loads of different ranges are independent).
__global__ void latent_merge_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out, const int* __restrict__ rows,
                                    const int* __restrict__ cu_q_lens, int nh, int splits) {
    __shared__ float weight[64];
    pdl_wait();
    const int n = blockIdx.y, h = blockIdx.x;
    const int tok = cu_q_lens[rows[n]];
    const float* base = scratch + ((size_t)n * splits * nh + h) * (RANK + 2);
    const size_t step = (size_t)nh * (RANK + 2);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m[2], l[2];
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int s = lane + 32 * i;
            m[i] = s < splits ? base[s * step + RANK] : -INFINITY;
            l[i] = s < splits ? base[s * step + RANK + 1] : 0.0f;
            M = fmaxf(M, m[i]);
        }
        M = warp_max(M);
        float e[2], L = 0.0f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            e[i] = m[i] == -INFINITY ? 0.0f : expf(m[i] - M);
            L += l[i] * e[i];
        }
        // the sum over the ranges in a fixed order
        float total = 0.0f;
        for (int s = 0; s < splits; ++s) total += __shfl_sync(0xffffffffu, (s < 32 ? l[0] * e[0] : l[1] * e[1]), s & 31);
        const float inv = total > 0.0f ? 1.0f / total : 0.0f;
#pragma unroll
        for (int i = 0; i < 2; ++i)
            if (lane + 32 * i < splits) weight[lane + 32 * i] = e[i] * inv;
        (void)L;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < RANK; c += blockDim.x) {
        float acc = 0.0f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) acc += base[s * step + c] * weight[s];
        out[((size_t)tok * nh + h) * RANK + c] = __float2bfloat16_rn(acc);
    }
}

template <int RG, int BN, int STAGES = 2>
size_t smem_bytes(int rot) {
    const int widthp = (RANK + rot + 63) & ~63, ld = widthp + 8, BM = 16 * RG;
    return ((size_t)BM * ld + (size_t)STAGES * BN * ld + (size_t)BM * (BN + 8)) * 2 + (size_t)(WARPS / RG) * BM * 4;
}

template <int RG, int BN, int STAGES = 2>
int launch(const Args& a, int n_list, int max_q_len, cudaStream_t stream) {
    const size_t smem = smem_bytes<RG, BN, STAGES>(a.rot);
    static size_t allowed = 0;
    if (smem > allowed) {
        if (cudaFuncSetAttribute(latent_attention_tc_kernel<RG, BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            LLME_REFUSE("latent attention: rows of %d values need %zu bytes of shared memory", RANK + a.rot, smem);
        }
        allowed = smem;
    }
    const int BM = 16 * RG;
    dim3 grid(((long long)max_q_len * a.nh + BM - 1) / BM, n_list, a.splits);
    llme_launch(latent_attention_tc_kernel<RG, BN, STAGES>, grid, dim3(WARPS * 32), smem, stream, a);
    LLME_LAUNCH_STATUS();
}

}  // namespace

// Whether rows of RANK + rot values fit the kernel (shared memory of the wider configuration).
LLME_API int llme_latent_attention_tc_fits(int rot) {
    if (rot < 0 || (RANK + rot) % 8) return 0;
    return smem_bytes<2, 64>(rot) <= 227u * 1024 ? 1 : 0;
}

// Scratch floats for `n_rows` requests of single tokens with `splits` blocks each.
LLME_API long long llme_latent_attention_scratch_floats(int n_rows, int nh, int splits) {
    return splits <= 1 ? 0 : (long long)n_rows * splits * nh * (RANK + 2);
}

// Requests `rows` of the step (indices into cu_q_lens / ctx_lens), each with any number of new tokens up to
// `max_q_len`.  `splits` > 1 only for requests of single tokens: their keys are cut into that many ranges.
LLME_API int llme_latent_attention_tc(const LlmeFastAttnArgs* f, const float* sink, int rot, int max_q_len, cudaStream_t stream) {
    if (f->n_rows <= 0 || max_q_len <= 0) return 0;
    if (!f->q || !f->cache || !f->out || !f->rows || !f->cu_q_lens || !f->ctx_lens || !f->table_rows || !f->block_tables)
        LLME_REFUSE("latent attention: null pointer");
    if (!llme_latent_attention_tc_fits(rot)) LLME_REFUSE("latent attention: rows of %d + %d values do not fit this kernel", RANK, rot);
    const int splits = f->splits < 1 ? 1 : f->splits;
    if (splits > 1 && (max_q_len != 1 || !f->scratch)) LLME_REFUSE("latent attention: splits need single tokens and scratch memory");
    if (f->n_rows > 65535 || splits > 64) LLME_REFUSE("latent attention: too many requests or splits for one launch");
    Args a = {(const __nv_bfloat16*)f->q, (const __nv_bfloat16*)f->cache, (__nv_bfloat16*)f->out, sink, f->rows, f->cu_q_lens, f->ctx_lens,
              f->table_rows, f->block_tables, f->scratch, f->max_blocks, f->nh, rot, f->page_size, splits, f->scale, f->window};
    int rc;
    if ((long long)max_q_len * f->nh <= 16) rc = launch<1, 64>(a, f->n_rows, max_q_len, stream);
    else if ((long long)max_q_len * f->nh <= 32) rc = launch<2, 64>(a, f->n_rows, max_q_len, stream);
    // prompt portions: 64 rows x 32 keys.  Measured on a 2,048-token prompt with rows of 512 + 64 (four layers, whole
    // step): 3.80 ms with this shape, 3.99 ms with 32 x 32, 4.22 ms with 32 x 64, 4.17 / 3.98 ms with a single key stage
    // and two or three blocks an SM: the time is in the fragments every warp re-reads from shared memory per key tile,
    // which no tile shape of a warp-level product removes.
    else rc = launch<4, 32>(a, f->n_rows, max_q_len, stream);
    if (rc || splits == 1) return rc;
    llme_launch(latent_merge_kernel, dim3(f->nh, f->n_rows), dim3(RANK >= 512 ? 256 : (RANK >= 256 ? 128 : 64)), 0, stream, (const float*)f->scratch,
                (__nv_bfloat16*)f->out, f->rows, f->cu_q_lens, f->nh, splits);
    LLME_LAUNCH_STATUS();
}

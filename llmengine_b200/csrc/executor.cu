// The step executor: walks a plan (the model's operation records) for one step and launches, per record, the kernel
// that serves the step's shape.  Host code only; the interface and the ideas are in
// include/llmengine_b200/executor.h.  The kernels live in libraries of their own and are reached through entry
// points registered by name, so this file knows their argument blocks (kernel_args.h) but not their code.
//
// Library matrix products (bfloat16 products of 17 to 127 tokens, and larger ones whose tiles would not fill the
// GPU) go to cuBLAS, as the reference's do (src/runtime/kernels/cuda_kernels.cu:892-908).  cuBLAS is not linked:
// the copy already in the process (PyTorch's) is looked up at run time, and the caller's handle is used when the
// step brings one, so that a captured step and an eager one take the same library path.
#include <cublas_v2.h>
#include <dlfcn.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "kernel_args.h"
#include "llmengine_b200/executor.h"

#define LLME_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// entry points of the kernel libraries
typedef int (*EmbeddingFn)(const int*, const void*, int, float*, int, int, int, cudaStream_t);
typedef int (*RmsNormFn)(float*, const void*, int, const void*, int, void*, int, const int*, int, int, float, cudaStream_t);
typedef int (*QkvPostFn)(const LlmeQkvArgs*, int, int, cudaStream_t);
typedef int (*SwigluFn)(const void*, int, void*, int, int, int, cudaStream_t);
typedef int (*GemmF32Fn)(const float*, const void*, int, float*, int, int, int, long long, long long, long long, cudaStream_t);
typedef int (*GemmBf16Fn)(const void*, long long, const void*, long long, void*, int, long long, int, int, int, cudaStream_t);
typedef int (*GemmTcSwigluFn)(const void*, long long, const void*, long long, void*, long long, int, int, int, cudaStream_t);
typedef int (*AttnPlainFn)(const LlmeAttnArgs*, int, cudaStream_t);
typedef int (*AttnPortionFn)(const LlmeFastAttnArgs*, int, cudaStream_t);
typedef int (*AttnDecodeFn)(const LlmeFastAttnArgs*, cudaStream_t);
typedef int (*AttnDecodeFusedFn)(const LlmeFastAttnArgs*, const LlmeFusedQkv*, cudaStream_t);
typedef long long (*AttnScratchFn)(int, int, int);
typedef int (*AttnTcFn)(const void*, long long, long long, const LlmeTcAttnArgs*, int, cudaStream_t);
typedef const char* (*LastErrorFn)();
typedef int (*GemmActFn)(const void*, long long, const void*, long long, void*, int, long long, int, int, int, int, float, float, cudaStream_t);
typedef int (*XieluFn)(const void*, long long, void*, long long, int, int, int, float, float, cudaStream_t);
typedef int (*SigmoidMulFn)(const void*, long long, const void*, long long, void*, long long, int, int, int, cudaStream_t);
typedef int (*ResidualAddFn)(float*, const void*, const void*, int, void*, int, int, int, cudaStream_t);
typedef int (*GeluGatherMulFn)(const void*, long long, int, const int*, const void*, int, long long, int, int, void*, long long, int, int, cudaStream_t);
typedef int (*RmsNormAddFn)(float*, const float*, const void*, int, int, int, float, cudaStream_t);
typedef int (*LatentPostFn)(const LlmeLatentPostArgs*, int, cudaStream_t);
typedef int (*LatentAttnPlainFn)(const LlmeLatentAttnArgs*, int, cudaStream_t);
typedef int (*LatentAttnTcFn)(const LlmeFastAttnArgs*, const float*, int, int, cudaStream_t);
typedef int (*LatentFitsFn)(int);
typedef int (*PostNormFn)(float*, const void*, int, const void*, int, void*, int, int, int, float, int, cudaStream_t);
typedef int (*GatedActFn)(const void*, long long, void*, long long, int, int, int, int, float, float, cudaStream_t);
typedef int (*GemmGatedFn)(const void*, long long, const void*, long long, void*, int, long long, int, int, int, int, float, float, cudaStream_t);
typedef int (*WindowPostFn)(const LlmeWindowPostArgs*, int, cudaStream_t);
typedef int (*WindowAttnPlainFn)(const LlmeWindowAttnArgs*, int, cudaStream_t);
typedef int (*WindowAttnTcFn)(const LlmeWindowFastArgs*, int, int, cudaStream_t);
typedef int (*MoeRouteFn)(const LlmeMoeRouteArgs*, cudaStream_t);
typedef int (*GroupedFn)(const LlmeGroupedArgs*, int, int, int, cudaStream_t);
typedef int (*MoeCombineFn)(const float*, long long, const float*, const float*, float*, int, int, int, cudaStream_t);
typedef int (*EmbeddingScaledFn)(const int*, const void*, int, float*, int, int, int, float, cudaStream_t);
typedef int (*SigmoidMulScaledFn)(const void*, long long, const void*, long long, void*, long long, int, int, int, float, cudaStream_t);
typedef int (*GatedActBiasFn)(const void*, long long, void*, long long, int, int, int, int, float, float, const float*, cudaStream_t);
typedef int (*BiasAddFn)(void*, long long, int, const float*, int, int, cudaStream_t);
typedef int (*ShortConvFn)(const LlmeShortConvArgs*, int, cudaStream_t);
typedef int (*RotateFn)(const LlmeRotateArgs*, cudaStream_t);
typedef int (*RecurrenceFn)(const LlmeRecurrenceArgs*, cudaStream_t);
typedef int (*GatedNormFn)(const LlmeGatedNormArgs*, cudaStream_t);
typedef int (*RmsNormPairFn)(float*, const void*, int, const void*, int, void*, int, const int*, int, int, float, const void*, void*, cudaStream_t);
typedef int (*SigmoidMulGroupedFn)(const void*, long long, const void*, long long, void*, long long, int, int, int, float, int, cudaStream_t);
typedef int (*ResidualAddScaledFn)(float*, const void*, const void*, int, void*, int, int, int, const float*, const float*, cudaStream_t);
typedef int (*MoeCombineGatedFn)(const float*, long long, const float*, const float*, float*, int, int, int, const float*, long long, cudaStream_t);
typedef int (*RowNormFn)(const void*, long long, int, const void*, int, void*, long long, int, int, int, float, cudaStream_t);
typedef int (*ExpGatesFn)(const LlmeExpGatesArgs*, int, cudaStream_t);
typedef int (*GemmF32BatchedFn)(const float*, const void*, int, float*, int, int, int, long long, long long, long long, int, long long,
                                long long, long long, cudaStream_t);

struct Blas {
    void* lib = nullptr;
    cublasStatus_t (*create)(cublasHandle_t*) = nullptr;
    cublasStatus_t (*destroy)(cublasHandle_t) = nullptr;
    cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
    cublasStatus_t (*set_math)(cublasHandle_t, cublasMath_t) = nullptr;
    cublasStatus_t (*set_workspace)(cublasHandle_t, void*, size_t) = nullptr;
    cublasStatus_t (*gemm_ex)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                              cudaDataType, int, const void*, cudaDataType, int, const void*, void*, cudaDataType, int,
                              cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
    cublasStatus_t (*gemm_batched)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                                   cudaDataType, int, long long, const void*, cudaDataType, int, long long, const void*, void*,
                                   cudaDataType, int, long long, int, cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
    bool load() {
        if (lib) return gemm_ex != nullptr;
        for (const char* name : {"libcublas.so.12", "libcublas.so"}) {
            lib = dlopen(name, RTLD_NOW | RTLD_NOLOAD);          // the copy the process already has
            if (lib) break;
        }
        if (!lib)
            for (const char* name : {"libcublas.so.12", "libcublas.so", "/usr/local/cuda/lib64/libcublas.so.12", "/usr/local/cuda/lib64/libcublas.so"}) {
                lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
                if (lib) break;
            }
        if (!lib) return false;
        create = (decltype(create))dlsym(lib, "cublasCreate_v2");
        destroy = (decltype(destroy))dlsym(lib, "cublasDestroy_v2");
        set_stream = (decltype(set_stream))dlsym(lib, "cublasSetStream_v2");
        set_math = (decltype(set_math))dlsym(lib, "cublasSetMathMode");
        set_workspace = (decltype(set_workspace))dlsym(lib, "cublasSetWorkspace_v2");
        gemm_ex = (decltype(gemm_ex))dlsym(lib, "cublasGemmEx");
        gemm_batched = (decltype(gemm_batched))dlsym(lib, "cublasGemmStridedBatchedEx");
        return create && destroy && set_stream && set_math && set_workspace && gemm_ex && gemm_batched;
    }
};

}  // namespace

struct LlmeExecutor {
    int device = 0, sms = 148;
    std::map<std::string, void*> entry;
    std::map<std::string, std::string> chosen;
    std::string error;
    long long launches = 0;
    Blas blas;
    cublasHandle_t own_handle = nullptr;
    void* own_workspace = nullptr;

    void* find(const std::string& name) const {
        auto it = entry.find(name);
        return it == entry.end() ? nullptr : it->second;
    }
    void* find_hd(const char* name, int hd) const { return find(std::string(name) + "/" + std::to_string(hd)); }
    const std::string& choice(const char* op) { return chosen[op]; }
    int fail(const char* fmt, ...) {
        char buf[768];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        error = buf;
        return -1;
    }
    // a kernel library's launcher returned rc: count the launch, keep the library's message on failure
    int launched(int rc, const char* kernel) {
        ++launches;
        if (rc == 0) return 0;
        const char* msg = "";
        std::string base(kernel);
        if (auto* f = (LastErrorFn)find("error/" + base)) msg = f();
        if (!msg || !*msg) msg = rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "refused";
        error = std::string(kernel) + ": " + msg + " (code " + std::to_string(rc) + ")";
        return rc;
    }
};

struct LlmePlan {
    LlmeExecutor* ex;
    struct Record {
        int kind;
        std::vector<unsigned char> bytes;
    };
    std::vector<Record> records;
};

namespace {

size_t record_size(int kind) {
    switch (kind) {
        case LLME_OP_EMBEDDING: return sizeof(LlmeEmbeddingOp);
        case LLME_OP_RMSNORM: return sizeof(LlmeRmsNormOp);
        case LLME_OP_LINEAR: return sizeof(LlmeLinearOp);
        case LLME_OP_LINEAR_SWIGLU: return sizeof(LlmeLinearSwigluOp);
        case LLME_OP_QKV_POST: return sizeof(LlmeQkvPostOp);
        case LLME_OP_ATTEND: return sizeof(LlmeAttendOp);
        case LLME_OP_ATTENTION: return sizeof(LlmeAttentionOp);
        case LLME_OP_CALL: return sizeof(LlmeCallOp);
        case LLME_OP_LINEAR_ACT: return sizeof(LlmeLinearActOp);
        case LLME_OP_POINTWISE: return sizeof(LlmePointwiseOp);
        case LLME_OP_BATCHED_LINEAR: return sizeof(LlmeBatchedLinearOp);
        case LLME_OP_RESIDUAL_ADD: return sizeof(LlmeResidualAddOp);
        case LLME_OP_LATENT_ATTENTION: return sizeof(LlmeLatentAttentionOp);
        case LLME_OP_TOKEN_SIDE: return sizeof(LlmeTokenSideOp);
        case LLME_OP_POSTNORM: return sizeof(LlmePostNormOp);
        case LLME_OP_WINDOW_ATTENTION: return sizeof(LlmeWindowAttentionOp);
        case LLME_OP_MOE_ROUTE: return sizeof(LlmeMoeRouteOp);
        case LLME_OP_GROUPED_LINEAR: return sizeof(LlmeGroupedLinearOp);
        case LLME_OP_MOE_COMBINE: return sizeof(LlmeMoeCombineOp);
        case LLME_OP_SHORT_CONV: return sizeof(LlmeShortConvOp);
        case LLME_OP_ROTATE: return sizeof(LlmeRotateOp);
        case LLME_OP_RECURRENCE: return sizeof(LlmeRecurrenceOp);
        case LLME_OP_GATED_NORM: return sizeof(LlmeGatedNormOp);
        case LLME_OP_ROW_NORM: return sizeof(LlmeRowNormOp);
        case LLME_OP_EXP_GATES: return sizeof(LlmeExpGatesOp);
    }
    return 0;
}
const char* kind_name(int kind) {
    static const char* names[] = {"?", "embedding", "rmsnorm", "linear", "linear_swiglu", "qkv_post", "attend", "attention", "call",
                                  "linear_act", "pointwise", "batched_linear", "residual_add", "latent_attention", "token_side",
                                  "postnorm", "window_attention", "moe_route", "grouped_linear", "moe_combine", "short_conv", "rotate",
                                  "recurrence", "gated_norm", "row_norm", "exp_gates"};
    return kind >= 1 && kind <= 25 ? names[kind] : names[0];
}

constexpr int SKINNY_ROWS = 16;      // most rows the weight-streaming product takes (gemm_skinny.cu)

// Whether a product of M tokens goes to the weight-streaming kernel when the choice is "auto".  That kernel has one
// block per group of 16 weight rows (8 gate + 8 up rows with the activation), two blocks resident per SM: it wins
// against the library's product for up to 8 tokens when its blocks fill their waves (4096 rows: 256 blocks for 296
// places, 5.5 TB/s on 4096 x 12288 against 3.1), and loses when a second wave is nearly empty (5120 rows: 320 blocks,
// 4.5 TB/s on 5120 x 17408 against 5.6) or when 9 to 16 tokens double the operands it re-reads from L2 per block.
// Where its waves of 296 are badly filled the kernel has a lighter form with three blocks per SM (444 places: 6.1 TB/s
// on 5120 x 17408 / 25600, against 5.7 to 5.9 for the library); 7,168 rows (448 groups) fit neither and go to the library.
bool skinny_pays(const LlmeExecutor& ex, int M, long long row_groups) {
    const long long places = 2LL * ex.sms, waves = (row_groups + places - 1) / places;
    // 9 to 16 tokens: only where the row groups are one well-filled round (4,096 rows: 256 groups).  There the kernel
    // takes 8.0 / 20.0 us for 4096 x 4096 / 4096 x 12288 against 10.6 / 21.7 us; with more row groups, each re-reading
    // the tokens' operands, the library is ahead (6144 x 4096: 14.3 against 12.9 us; 24576 x 4096: 39.5 against 37.7).
    if (M > 8) return row_groups <= places && 10 * row_groups >= 8 * places;
    if (4 * row_groups <= places) return true;          // a small product is bound by its launch, not by its waves
    if (10 * row_groups >= 8 * waves * places) return true;
    // the kernel's lighter form, three blocks per SM: 444 places a round (gemm_skinny.cu chooses it by the same figures)
    const long long places3 = 3LL * ex.sms, waves3 = (row_groups + places3 - 1) / places3;
    return 10 * row_groups >= 7 * waves3 * places3;
}

bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr) {
    return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0;
}

// Whether a plain product of this size goes to this package's tcgen05 kernel rather than to cuBLAS when the choice is
// "auto".  The kernel walks over whole tiles: 256 x 256 per pair of SMs from 129 tokens and 129 columns on (128 x 256
// or 128 x 128 per SM below that).  128 tiles on 74 pairs take the time of two waves for 1.73 waves of work, and there
// cuBLAS, which has the same tiles but more shapes to choose from, is 4 % faster (2,048 tokens of the 8B shape: 53 / 75
// / 153 us for the output, q|k|v and down products against 51 / 72 / 156 us; at 8,192 tokens, where the waves are
// full, 194 / 289 / 704 us against 259 / 301 / 806 us).  "auto" takes the kernel when its last wave is at least 90 % full.
bool tc_fills_its_waves(const LlmeExecutor& ex, int M, int N) {
    const bool pairs = M > 128 && N > 128;
    const long long tiles = pairs ? (long long)((M + 255) / 256) * ((N + 255) / 256)
                                  : (long long)((M + 127) / 128) * ((N + (N > 128 ? 255 : 127)) / (N > 128 ? 256 : 128));
    const long long walkers = pairs ? ex.sms / 2 : ex.sms;
    const long long waves = (tiles + walkers - 1) / walkers;
    return 10 * tiles >= 9 * waves * walkers;
}

// One handle for the library products of this step: the caller's, or the executor's own.
int blas_handle(LlmeExecutor& ex, const LlmeStep& step, cudaStream_t stream, cublasHandle_t* out) {
    if (!ex.blas.load()) return ex.fail("linear: cuBLAS is not available in this process");
    cublasHandle_t h = (cublasHandle_t)step.blas;
    if (!h) {
        if (!ex.own_handle) {
            if (ex.blas.create(&ex.own_handle) != CUBLAS_STATUS_SUCCESS) return ex.fail("linear: cublasCreate failed");
            if (cudaMalloc(&ex.own_workspace, 32u << 20) == cudaSuccess) ex.blas.set_workspace(ex.own_handle, ex.own_workspace, 32u << 20);
        }
        h = ex.own_handle;
        ex.blas.set_stream(h, stream);
    }
    *out = h;
    return 0;
}

int cublas_product(LlmeExecutor& ex, const LlmeStep& step, const void* x, long long ldx, const void* w, long long ldw, void* out,
                   long long ldo, int out_dtype, int M, int N, int K, cudaStream_t stream) {
    cublasHandle_t h;
    if (int rc = blas_handle(ex, step, stream, &h)) return rc;
    // partial sums are never added in bfloat16: some shapes (a few tokens, an odd width) otherwise come out a
    // thousand rounding steps off
    ex.blas.set_math(h, (cublasMath_t)(CUBLAS_DEFAULT_MATH | CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION));
    const float alpha = 1.0f, beta = 0.0f;
    const cublasStatus_t st = ex.blas.gemm_ex(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, (int)ldw, x, CUDA_R_16BF,
                                              (int)ldx, &beta, out, out_dtype == LLME_DT_F32 ? CUDA_R_32F : CUDA_R_16BF, (int)ldo,
                                              CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    ex.blas.set_math(h, CUBLAS_DEFAULT_MATH);
    if (st != CUBLAS_STATUS_SUCCESS) return ex.fail("linear: cublasGemmEx failed with status %d for M=%d N=%d K=%d", (int)st, M, N, K);
    return 0;
}

int rows_of(const LlmeStep& s, int rows) { return rows == LLME_ROWS_LOGITS ? s.num_logit_rows : s.num_tokens; }

// out[M, n] = x[M, k] w[n, k]^T
int product(LlmeExecutor& ex, const LlmeStep& step, const void* x, long long ldx, int x_dtype, const void* w, long long ldw,
            int w_dtype, void* out, long long ldo, int out_dtype, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (x_dtype == LLME_DT_F32) {
        // the 32-bit path: this package's FMA kernel, never a reduced-precision mode
        auto* f = (GemmF32Fn)ex.find("gemm_f32");
        if (!f) return ex.fail("linear: no 32-bit product kernel is registered");
        if (out_dtype != LLME_DT_F32) return ex.fail("linear: a 32-bit product writes 32-bit output");
        return ex.launched(f((const float*)x, w, w_dtype, (float*)out, M, N, K, ldx, ldw, ldo, stream), "gemm_f32");
    }
    if (w_dtype != LLME_DT_BF16) return ex.fail("linear: bfloat16 inputs need bfloat16 weights");
    const std::string& how = ex.choice("linear");
    const bool operands_ok = K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && aligned16(x, w);
    const std::string& dec = ex.choice("linear.decode");
    if (how != "plain" && M <= SKINNY_ROWS && operands_ok && (dec == "skinny" || (dec == "auto" && skinny_pays(ex, M, (N + 15) / 16)))) {
        if (auto* f = (GemmBf16Fn)ex.find("gemm_skinny"))     // a handful of tokens: the weight-streaming kernel
            return ex.launched(f(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, stream), "gemm_skinny");
    }
    if (M >= 128 && operands_ok && N >= 8 && ldo >= N && (how == "tcgen05" || (how == "auto" && tc_fills_its_waves(ex, M, N)))) {
        if (auto* f = (GemmBf16Fn)ex.find("gemm_tc"))         // many tokens: the tcgen05 kernel
            return ex.launched(f(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, stream), "gemm_tc");
    }
    return cublas_product(ex, step, x, ldx, w, ldw, out, ldo, out_dtype, M, N, K, stream);
}

int op_embedding(LlmeExecutor& ex, const LlmeEmbeddingOp& o, const LlmeStep& s, cudaStream_t st) {
    if (o.scale != 1.0f) {
        auto* g = (EmbeddingScaledFn)ex.find("embedding_scaled");
        if (!g) return ex.fail("no kernel for a scaled embedding is registered");
        return ex.launched(g(s.token_ids, o.table, o.table_dtype, o.out, s.num_tokens, o.hidden, o.vocab, o.scale, st), "embedding");
    }
    auto* f = (EmbeddingFn)ex.find("embedding");
    if (!f) return ex.fail("no embedding kernel is registered");
    return ex.launched(f(s.token_ids, o.table, o.table_dtype, o.out, s.num_tokens, o.hidden, o.vocab, st), "embedding");
}

int op_rmsnorm(LlmeExecutor& ex, const LlmeRmsNormOp& o, const LlmeStep& s, cudaStream_t st) {
    auto* f = (RmsNormFn)ex.find("rmsnorm");
    if (!f) return ex.fail("no rmsnorm kernel is registered");
    const bool some = o.rows == LLME_ROWS_LOGITS;
    if (o.gain2) {
        auto* g = (RmsNormPairFn)ex.find("rmsnorm_pair");
        if (!g) return ex.fail("no rmsnorm kernel with a second gain is registered");
        return ex.launched(g(o.x, o.delta, o.delta_dtype, o.gain, o.gain_dtype, o.out, o.out_dtype, some ? s.logit_rows : nullptr,
                             rows_of(s, o.rows), o.size, o.eps, o.gain2, o.out2, st), "rmsnorm");
    }
    return ex.launched(f(o.x, o.delta, o.delta_dtype, o.gain, o.gain_dtype, o.out, o.out_dtype, some ? s.logit_rows : nullptr,
                         rows_of(s, o.rows), o.size, o.eps, st), "rmsnorm");
}

int op_linear(LlmeExecutor& ex, const LlmeLinearOp& o, const LlmeStep& s, cudaStream_t st) {
    if (rows_of(s, o.rows) <= 0) return 0;
    void* out = o.out ? o.out : (void*)s.logits;
    if (!out) return ex.fail("linear: the step has no place for its logits");
    if (int rc = product(ex, s, o.x, o.ldx, o.x_dtype, o.w, o.ldw, o.w_dtype, out, o.out ? o.ldo : o.n, o.out ? o.out_dtype : LLME_DT_F32,
                         rows_of(s, o.rows), o.n, o.k, st))
        return rc;
    if (!o.bias) return 0;
    auto* add = (BiasAddFn)ex.find("bias_add");
    if (!add) return ex.fail("linear: no kernel that adds a bias is registered");
    return ex.launched(add(out, o.out ? o.ldo : o.n, o.out ? o.out_dtype : LLME_DT_F32, o.bias, rows_of(s, o.rows), o.n, st), "bias_add");
}

int op_linear_swiglu(LlmeExecutor& ex, const LlmeLinearSwigluOp& o, const LlmeStep& s, cudaStream_t st) {
    const int M = s.num_tokens;
    if (M <= 0) return 0;
    // biases before the activation: the product with the activation kernel behind it, which adds them
    const bool fused = ex.choice("linear_swiglu") == "fused" && ex.choice("linear") != "plain" && o.dtype == LLME_DT_BF16 && !o.bias;
    const bool operands_ok = o.k % 8 == 0 && o.ldx % 8 == 0 && o.ldw % 8 == 0 && aligned16(o.x, o.w_gate_up);
    const std::string& dec = ex.choice("linear.decode");
    if (fused && M <= SKINNY_ROWS && operands_ok && (dec == "skinny" || (dec == "auto" && skinny_pays(ex, M, (o.inter + 7) / 8)))) {
        if (o.act != LLME_GATE_SILU) {
            if (auto* f = (GemmGatedFn)ex.find("gemm_skinny_gated"))
                return ex.launched(f(o.x, o.ldx, o.w_gate_up, o.ldw, o.out, LLME_DT_BF16, o.ldo, M, o.inter, o.k, o.act, o.p0, o.p1, st), "gemm_skinny_gated");
        } else if (auto* f = (GemmBf16Fn)ex.find("gemm_skinny_swiglu"))
            return ex.launched(f(o.x, o.ldx, o.w_gate_up, o.ldw, o.out, LLME_DT_BF16, o.ldo, M, o.inter, o.k, st), "gemm_skinny_swiglu");
    }
    // the tcgen05 kernel with the activation in its epilogue: its tile is 128 tokens x (128 gate + 128 up) rows; like
    // the plain product it is taken only when its last wave is nearly full (at 256 / 512 / 1,024 tokens of the 8B
    // shape the library product with the activation kernel behind it is faster)
    const std::string& how = ex.choice("linear");
    if (fused && M >= 128 && operands_ok && o.inter >= 8 && o.ldo % 8 == 0 && aligned16(o.out) &&
        (how == "tcgen05" || (how == "auto" && tc_fills_its_waves(ex, M, 2 * o.inter)))) {
        if (o.act != LLME_GATE_SILU) {
            if (auto* f = (GemmGatedFn)ex.find("gemm_tc_gated"))
                return ex.launched(f(o.x, o.ldx, o.w_gate_up, o.ldw, o.out, LLME_DT_BF16, o.ldo, M, o.inter, o.k, o.act, o.p0, o.p1, st), "gemm_tc_gated");
        } else if (auto* f = (GemmTcSwigluFn)ex.find("gemm_tc_swiglu"))
            return ex.launched(f(o.x, o.ldx, o.w_gate_up, o.ldw, o.out, o.ldo, M, o.inter, o.k, st), "gemm_tc_swiglu");
    }
    if (!o.gate_up) return ex.fail("linear_swiglu: the unfused form needs a workspace for gate|up");
    if (int rc = product(ex, s, o.x, o.ldx, o.dtype, o.w_gate_up, o.ldw, o.dtype, o.gate_up, 2LL * o.inter, o.dtype, M, 2 * o.inter, o.k, st))
        return rc;
    if (o.bias) {
        auto* g = (GatedActBiasFn)ex.find("gated_act_bias");
        if (!g) return ex.fail("no gated activation kernel with biases is registered");
        return ex.launched(g(o.gate_up, 2LL * o.inter, o.out, o.ldo, o.dtype, M, o.inter, o.act, o.p0, o.p1, o.bias, st), "gated_act");
    }
    if (o.act != LLME_GATE_SILU) {
        auto* g = (GatedActFn)ex.find("gated_act");
        if (!g) return ex.fail("no gated activation kernel is registered");
        return ex.launched(g(o.gate_up, 2LL * o.inter, o.out, o.ldo, o.dtype, M, o.inter, o.act, o.p0, o.p1, st), "gated_act");
    }
    auto* f = (SwigluFn)ex.find("swiglu");
    if (!f) return ex.fail("no swiglu kernel is registered");
    if (o.ldo != o.inter) return ex.fail("linear_swiglu: the unfused form writes dense rows");
    return ex.launched(f(o.gate_up, o.dtype, o.out, o.dtype, M, o.inter, st), "swiglu");
}

int op_qkv_post(LlmeExecutor& ex, const LlmeQkvPostOp& o, const LlmeStep& s, cudaStream_t st) {
    auto* f = (QkvPostFn)ex.find("qkv_post");
    if (!f) return ex.fail("no qkv_post kernel is registered");
    if (!o.q_out && !o.k_out && !o.cache) return 0;
    if (o.cache && (o.group < 0 || o.group >= s.num_groups)) return ex.fail("qkv_post: the step has no cache group %d", o.group);
    LlmeQkvArgs a = {};
    a.q_in = o.q_in; a.k_in = o.k_in; a.v_in = o.v_in;
    a.q_stride = o.q_stride; a.k_stride = o.k_stride; a.v_stride = o.v_stride;
    a.q_gain = o.q_gain; a.k_gain = o.k_gain; a.gain_dtype = o.gain_dtype; a.eps = o.eps;
    a.cos_sin = o.cos_sin; a.positions = s.positions; a.max_positions = o.max_positions;
    a.q_out = o.q_out; a.k_out = o.k_out; a.cache = o.cache;
    a.slot_mapping = o.cache ? s.groups[o.group].slot_mapping : nullptr;
    a.tokens = s.num_tokens; a.nh = o.nh; a.nkv = o.nkv; a.hd = o.hd;
    a.page_size = o.cache ? s.groups[o.group].page_size : 0;
    return ex.launched(f(&a, o.in_dtype, o.out_dtype, st), "qkv_post");
}

// Blocks per (request, key/value head) of the decode attention, chosen by what the kernel's time is made of.  A block
// streams its share of the keys at a rate of its own (about 27 GB/s: its warps' loads wait for one another), and
// needs about 6 us beside that, the time of some 300 keys; the blocks run in rounds of as many as the GPU holds at
// once.  Up to 8 splits are one thread-block cluster and merge through shared memory; the blocks of a cluster must find
// room in one GPC together, so the GPU holds fewer clusters than its SMs hold blocks (71 of four blocks, not 74; 93 of
// three, not 98: the kernel library says how many), and one cluster too many is a second round: 9 requests of 8
// key/value heads in clusters of four took 33 us a layer against 17 us for 8 requests, 19 us in clusters of three.
// More than 8 splits (at most 16) merge through scratch memory, where the block that finishes last adds the parts up,
// the dearer the more there are (batch 1, 8,200 keys: 15.1 us with 16 splits, 16.9 us with 37, 23.2 us with 64).
// Measured choices this reproduces: batch 1 / 8 / 9 / 12 / 16 / 24 / 40 at 2,048 keys: 8 / 4 / 3 / 2 / 2 / 1 / 3 splits.
typedef int (*AttnClustersFn)(int);

int decode_splits(const LlmeExecutor& ex, int requests, int nh, int nkv, int hd, int window, long long max_ctx) {
    const long long span = window > 0 && window < max_ctx ? window : max_ctx;
    const long long groups = (span + 63) / 64 + (window > 0 ? 1 : 0);      // 64-key groups of the longest context
    const int G = nh / nkv;
    const long long units = (long long)requests * nkv * ((G + 15) / 16);     // (request, key/value head, 16 query heads)
    auto* room = (AttnClustersFn)ex.find_hd("attention_decode_clusters", hd);
    long long best = 1, best_cost = -1;
    for (long long s = 1; s <= 16 && s <= groups; ++s) {
        long long held = 2LL * ex.sms;                                       // blocks the GPU holds at once
        if (s >= 2 && s <= 8 && room) {
            const int clusters = room((int)s);
            if (clusters > 0) held = s * clusters;
        }
        const long long rounds = (units * s + held - 1) / held;
        const long long keys = (groups + s - 1) / s * 64;
        const long long fixed = s <= 8 ? 300 : 300 + 25 * s;
        const long long cost = rounds * (keys + fixed) * (100 + 8 * (rounds - 1));      // later rounds are never quite full
        if (best_cost < 0 || cost < best_cost) { best = s; best_cost = cost; }
    }
    return (int)best;
}

bool fast_attention(LlmeExecutor& ex, int dtype, int hd) {
    return ex.choice("attention") == "fast" && dtype == LLME_DT_BF16 && hd % 16 == 0 && hd >= 16 && hd <= 128 &&
           ex.find_hd("attention_decode", hd) && ex.find_hd("attention_portion", hd);
}

void fill_fast(LlmeFastAttnArgs& a, const LlmeAttendOp& o, const LlmeStep& s, const int* rows, int n_rows, int splits) {
    const LlmeStepGroup& g = s.groups[o.group];
    a.q = o.q; a.cache = o.cache; a.out = o.out; a.rows = rows; a.cu_q_lens = s.cu_q_lens; a.ctx_lens = s.ctx_lens;
    a.table_rows = s.state_slots; a.block_tables = g.block_tables; a.scratch = o.scratch;
    a.max_blocks = g.max_blocks; a.n_rows = n_rows; a.nh = o.nh; a.nkv = o.nkv; a.page_size = g.page_size; a.window = o.window;
    a.splits = splits; a.scale = o.scale;
}

int scratch_check(LlmeExecutor& ex, const LlmeAttendOp& o, int n_rows, int splits) {
    if (splits <= 1) return 0;
    auto* need = (AttnScratchFn)ex.find_hd("attention_decode_scratch", o.hd);
    const long long floats = need ? need(n_rows, o.nh, splits) : 65536 + (long long)n_rows * o.nh * splits * (o.hd + 2);
    if (!o.scratch || floats > o.scratch_floats)
        return ex.fail("attention: %d requests x %d splits need %lld scratch values, the record has %lld", n_rows, splits, floats, o.scratch_floats);
    return 0;
}

int op_attend(LlmeExecutor& ex, const LlmeAttendOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    if (o.group < 0 || o.group >= s.num_groups) return ex.fail("attention: the step has no cache group %d", o.group);
    const LlmeStepGroup& g = s.groups[o.group];
    if (!fast_attention(ex, o.dtype, o.hd)) {
        auto* f = (AttnPlainFn)ex.find("attention_plain");
        if (!f) return ex.fail("no plain attention kernel is registered");
        LlmeAttnArgs a = {o.q, o.cache, o.out, s.positions, s.token_request, g.block_tables, g.max_blocks, s.num_tokens, o.nh, o.nkv,
                          o.hd, g.page_size, o.window, o.scale};
        return ex.launched(f(&a, o.dtype, st), "attention_plain");
    }
    if (s.num_portion > 0) {
        const int G = o.nh / o.nkv, ps = g.page_size;
        const bool pages_ok = ps >= 8 && (ps <= 128 ? 128 % ps == 0 : ps % 128 == 0);
        auto* tc = (AttnTcFn)ex.find_hd("attention_tc", o.hd);
        if (tc && ex.choice("attention.portion") == "tcgen05" && (o.hd == 64 || o.hd == 128) && pages_ok && 128 % G == 0) {
            LlmeTcAttnArgs a = {o.out, o.cache, s.portion_rows, s.cu_q_lens, s.ctx_lens, s.state_slots, g.block_tables, g.max_blocks,
                                s.num_portion, o.nh, o.nkv, ps, o.window, o.scale};
            if (int rc = ex.launched(tc(o.q, s.num_tokens, o.cache_rows, &a, s.max_portion_len, st), "attention_tc")) return rc;
        } else {
            LlmeFastAttnArgs a = {};
            fill_fast(a, o, s, s.portion_rows, s.num_portion, 1);
            auto* f = (AttnPortionFn)ex.find_hd("attention_portion", o.hd);
            if (int rc = ex.launched(f(&a, s.max_portion_len, st), "attention_portion")) return rc;
        }
    }
    if (s.num_decode > 0) {
        const int splits = decode_splits(ex, s.num_decode, o.nh, o.nkv, o.hd, o.window, s.max_decode_ctx);
        if (int rc = scratch_check(ex, o, s.num_decode, splits)) return rc;
        LlmeFastAttnArgs a = {};
        fill_fast(a, o, s, s.decode_rows, s.num_decode, splits);
        auto* f = (AttnDecodeFn)ex.find_hd("attention_decode", o.hd);
        if (int rc = ex.launched(f(&a, st), "attention_decode")) return rc;
    }
    return 0;
}

int op_attention(LlmeExecutor& ex, const LlmeAttentionOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    const LlmeAttendOp& at = o.attend;
    auto* fused = (AttnDecodeFusedFn)ex.find_hd("attention_decode_fused", at.hd);
    // a step of single new tokens: norm, rotation and cache write happen inside the attention kernel
    if (fused && fast_attention(ex, at.dtype, at.hd) && ex.choice("attention.decode") == "fused" && s.num_portion == 0 &&
        s.num_decode == s.num_tokens && at.hd % 4 == 0 && o.qkv_stride % 2 == 0 &&
        (((uintptr_t)o.qkv | (uintptr_t)o.post.q_gain | (uintptr_t)o.post.k_gain | (uintptr_t)o.post.cos_sin) & 7) == 0) {
        if (at.group < 0 || at.group >= s.num_groups) return ex.fail("attention: the step has no cache group %d", at.group);
        const int splits = decode_splits(ex, s.num_decode, at.nh, at.nkv, at.hd, at.window, s.max_decode_ctx);
        if (int rc = scratch_check(ex, at, s.num_decode, splits)) return rc;
        LlmeFastAttnArgs a = {};
        fill_fast(a, at, s, s.decode_rows, s.num_decode, splits);
        a.q = nullptr;
        LlmeFusedQkv f = {o.qkv, o.qkv_stride, o.post.q_gain, o.post.k_gain, o.post.gain_dtype, o.post.eps,
                          o.rotary ? o.post.cos_sin : nullptr, o.rotary ? o.post.max_positions : 0, o.post.cache ? 1 : 0};
        return ex.launched(fused(&a, &f, st), "attention_decode_fused");
    }
    if (int rc = op_qkv_post(ex, o.post, s, st)) return rc;
    return op_attend(ex, at, s, st);
}

int op_linear_act(LlmeExecutor& ex, const LlmeLinearActOp& o, const LlmeStep& s, cudaStream_t st) {
    const int M = s.num_tokens;
    if (M <= 0) return 0;
    const LlmeLinearOp& p = o.product;
    if (o.act != LLME_ACT_XIELU) return ex.fail("linear_act: unknown activation %d", o.act);
    // a handful of tokens: the weight-streaming product carries the activation in its epilogue (same rule as the plain product)
    const std::string& dec = ex.choice("linear.decode");
    if (p.x_dtype == LLME_DT_BF16 && p.w_dtype == LLME_DT_BF16 && ex.choice("linear") != "plain" && ex.choice("linear_swiglu") == "fused" &&
        M <= SKINNY_ROWS && p.k % 8 == 0 && p.ldx % 8 == 0 && p.ldw % 8 == 0 && aligned16(p.x, p.w) &&
        (dec == "skinny" || (dec == "auto" && skinny_pays(ex, M, (p.n + 15) / 16)))) {
        if (auto* f = (GemmActFn)ex.find("gemm_skinny_act"))
            return ex.launched(f(p.x, p.ldx, p.w, p.ldw, o.out, p.out_dtype, o.ldo, M, p.n, p.k, o.act, o.p0, o.p1, st), "gemm_skinny_act");
    }
    // many tokens: the tcgen05 product with the activation in its epilogue, where the plain product would take that kernel
    const std::string& how = ex.choice("linear");
    if (p.x_dtype == LLME_DT_BF16 && p.w_dtype == LLME_DT_BF16 && ex.choice("linear_swiglu") == "fused" && M >= 128 && p.k % 8 == 0 &&
        p.ldx % 8 == 0 && p.ldw % 8 == 0 && aligned16(p.x, p.w) && p.n >= 8 && o.ldo >= p.n &&
        (how == "tcgen05" || (how == "auto" && tc_fills_its_waves(ex, M, p.n)))) {
        if (auto* f = (GemmActFn)ex.find("gemm_tc_act"))
            return ex.launched(f(p.x, p.ldx, p.w, p.ldw, o.out, p.out_dtype, o.ldo, M, p.n, p.k, o.act, o.p0, o.p1, st), "gemm_tc_act");
    }
    if (!p.out) return ex.fail("linear_act: the product needs its workspace");
    if (int rc = product(ex, s, p.x, p.ldx, p.x_dtype, p.w, p.ldw, p.w_dtype, p.out, p.ldo, p.out_dtype, M, p.n, p.k, st)) return rc;
    auto* f = (XieluFn)ex.find("xielu");
    if (!f) return ex.fail("no xielu kernel is registered");
    return ex.launched(f(p.out, p.ldo, o.out, o.ldo, p.out_dtype, M, p.n, o.p0, o.p1, st), "xielu");
}

int op_pointwise(LlmeExecutor& ex, const LlmePointwiseOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    if (o.what != LLME_POINTWISE_SIGMOID_MUL) return ex.fail("pointwise: unknown operation %d", o.what);
    if (o.group > 1) {
        auto* g = (SigmoidMulGroupedFn)ex.find("sigmoid_mul_grouped");
        if (!g) return ex.fail("no sigmoid_mul kernel with one gate per group of columns is registered");
        return ex.launched(g(o.a, o.lda, o.b, o.ldb, o.out, o.ldo, o.dtype, s.num_tokens, o.cols, o.scale, o.group, st), "sigmoid_mul");
    }
    if (o.scale != 1.0f) {
        auto* g = (SigmoidMulScaledFn)ex.find("sigmoid_mul_scaled");
        if (!g) return ex.fail("no scaled sigmoid_mul kernel is registered");
        return ex.launched(g(o.a, o.lda, o.b, o.ldb, o.out, o.ldo, o.dtype, s.num_tokens, o.cols, o.scale, st), "sigmoid_mul");
    }
    auto* f = (SigmoidMulFn)ex.find("sigmoid_mul");
    if (!f) return ex.fail("no sigmoid_mul kernel is registered");
    return ex.launched(f(o.a, o.lda, o.b, o.ldb, o.out, o.ldo, o.dtype, s.num_tokens, o.cols, st), "sigmoid_mul");
}

int op_batched_linear(LlmeExecutor& ex, const LlmeBatchedLinearOp& o, const LlmeStep& s, cudaStream_t st) {
    const int M = s.num_tokens;
    if (M <= 0 || o.batch <= 0) return 0;
    if (o.x_dtype == LLME_DT_F32) {
        auto* f = (GemmF32BatchedFn)ex.find("gemm_f32_batched");
        if (!f) return ex.fail("batched_linear: no 32-bit batched product kernel is registered");
        if (o.out_dtype != LLME_DT_F32) return ex.fail("batched_linear: a 32-bit product writes 32-bit output");
        return ex.launched(f((const float*)o.x, o.w, o.w_dtype, (float*)o.out, M, o.n, o.k, o.ldx, o.ldw, o.ldo, o.batch, o.x_member,
                             o.w_member, o.out_member, st), "gemm_f32");
    }
    if (o.w_dtype != LLME_DT_BF16) return ex.fail("batched_linear: bfloat16 inputs need bfloat16 weights");
    cublasHandle_t h;
    if (int rc = blas_handle(ex, s, st, &h)) return rc;
    ex.blas.set_math(h, (cublasMath_t)(CUBLAS_DEFAULT_MATH | CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION));
    const float alpha = 1.0f, beta = 0.0f;
    const cublasStatus_t rc = ex.blas.gemm_batched(h, CUBLAS_OP_T, CUBLAS_OP_N, o.n, M, o.k, &alpha, o.w, CUDA_R_16BF, (int)o.ldw, o.w_member,
                                                   o.x, CUDA_R_16BF, (int)o.ldx, o.x_member, &beta, o.out,
                                                   o.out_dtype == LLME_DT_F32 ? CUDA_R_32F : CUDA_R_16BF, (int)o.ldo, o.out_member, o.batch,
                                                   CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    ex.blas.set_math(h, CUBLAS_DEFAULT_MATH);
    if (rc != CUBLAS_STATUS_SUCCESS)
        return ex.fail("batched_linear: cublasGemmStridedBatchedEx failed with status %d for M=%d N=%d K=%d batch=%d", (int)rc, M, o.n, o.k, o.batch);
    return 0;
}

int op_residual_add(LlmeExecutor& ex, const LlmeResidualAddOp& o, const LlmeStep& s, cudaStream_t st) {
    if (o.a_scale || o.b_scale) {
        auto* g = (ResidualAddScaledFn)ex.find("residual_add_scaled");
        if (!g) return ex.fail("no residual_add kernel with scale vectors is registered");
        return ex.launched(g(o.x, o.a, o.b, o.dtype, nullptr, 0, s.num_tokens, o.size, o.a_scale, o.b_scale, st), "residual_add");
    }
    auto* f = (ResidualAddFn)ex.find("residual_add");
    if (!f) return ex.fail("no residual_add kernel is registered");
    return ex.launched(f(o.x, o.a, o.b, o.dtype, nullptr, 0, s.num_tokens, o.size, st), "residual_add");
}

// Key ranges per request for single tokens over a latent cache: as many blocks as the GPU has SMs, no range shorter
// than two key tiles, at most 32.  A request's heads are one tile of rows per 32 heads.
int latent_splits(const LlmeExecutor& ex, int requests, int nh, long long max_ctx, int window) {
    if (window > 0 && max_ctx > window) max_ctx = window;      // a token reads no more keys than its window holds
    const long long row_tiles = (nh + 31) / 32, bn = nh <= 32 ? 64 : 32;
    const long long tiles = (max_ctx + bn - 1) / bn;
    long long s = ex.sms / (requests * row_tiles);
    if (s > tiles / 2) s = tiles / 2;
    if (s > 32) s = 32;
    return s < 1 ? 1 : (int)s;
}

int op_latent_attention(LlmeExecutor& ex, const LlmeLatentAttentionOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    if (o.group < 0 || o.group >= s.num_groups) return ex.fail("latent attention: the step has no cache group %d", o.group);
    const LlmeStepGroup& g = s.groups[o.group];
    auto* post = (LatentPostFn)ex.find("latent_post");
    if (!post) return ex.fail("no latent_post kernel is registered");
    LlmeLatentPostArgs p = {};
    p.kv_in = o.kv_in; p.kv_stride = o.kv_stride; p.q_rot = o.q_rot; p.q_rot_stride = o.q_rot_stride; p.q_rot_head_stride = o.q_rot_head_stride;
    p.c_gain = o.c_gain; p.gain_dtype = o.gain_dtype; p.eps = o.eps; p.inv_freq = o.inv_freq; p.rot_dims = o.rot_dims;
    p.positions = s.positions; p.q = o.q; p.cache = o.cache; p.slot_mapping = g.slot_mapping;
    p.tokens = s.num_tokens; p.nh = o.nh; p.rank = o.rank; p.rot = o.rot; p.interleaved = o.interleaved;
    if (int rc = ex.launched(post(&p, o.dtype, st), "latent_post")) return rc;
    // bfloat16 with a latent size the tensor-core kernel is built for: prompt portions in one launch, single tokens in
    // another whose requests may be cut into several key ranges
    auto* tc = (LatentAttnTcFn)ex.find_hd("latent_attention_tc", o.rank);
    auto* fits = (LatentFitsFn)ex.find_hd("latent_attention_tc_fits", o.rank);
    if (tc && fits && o.dtype == LLME_DT_BF16 && ex.choice("attention") == "fast" && fits(o.rot)) {
        LlmeFastAttnArgs f = {};
        f.q = o.q; f.cache = o.cache; f.out = o.out; f.cu_q_lens = s.cu_q_lens; f.ctx_lens = s.ctx_lens; f.table_rows = s.state_slots;
        f.block_tables = g.block_tables; f.scratch = o.scratch; f.max_blocks = g.max_blocks; f.nh = o.nh; f.nkv = 1;
        f.page_size = g.page_size; f.scale = o.scale; f.window = o.window;
        if (s.num_portion > 0) {
            f.rows = s.portion_rows; f.n_rows = s.num_portion; f.splits = 1;
            if (int rc = ex.launched(tc(&f, o.sink, o.rot, s.max_portion_len, st), "latent_attention_tc")) return rc;
        }
        if (s.num_decode > 0) {
            f.rows = s.decode_rows; f.n_rows = s.num_decode;
            f.splits = latent_splits(ex, s.num_decode, o.nh, s.max_decode_ctx, o.window);
            if (f.splits > 1 && (!o.scratch || (long long)s.num_decode * f.splits * o.nh * (o.rank + 2) > o.scratch_floats)) f.splits = 1;
            if (int rc = ex.launched(tc(&f, o.sink, o.rot, 1, st), "latent_attention_tc")) return rc;
            if (f.splits > 1) ++ex.launches;
        }
        return 0;
    }
    auto* plain = (LatentAttnPlainFn)ex.find("latent_attention_plain");
    if (!plain) return ex.fail("no latent attention kernel is registered");
    LlmeLatentAttnArgs a = {o.q, o.cache, o.out, o.sink, s.positions, s.token_request, g.block_tables, g.max_blocks, s.num_tokens,
                            o.nh, o.rank, o.rot, g.page_size, o.scale, o.window};
    return ex.launched(plain(&a, o.dtype, st), "latent_attention_plain");
}

int op_token_side(LlmeExecutor& ex, const LlmeTokenSideOp& o, const LlmeStep& s, cudaStream_t st) {
    const int M = s.num_tokens;
    if (M <= 0) return 0;
    auto* add = (ResidualAddFn)ex.find("residual_add");
    auto* gate = (GeluGatherMulFn)ex.find("gelu_gather_mul");
    auto* norm = (RmsNormAddFn)ex.find("rmsnorm_add");
    if (!add || !gate || !norm) return ex.fail("the kernels of the token side input are not registered");
    // the stream itself is the gate's input: in the 32-bit path as it is, else a copy in the type of the products
    const bool copy = o.act_dtype != LLME_DT_F32;
    if (int rc = ex.launched(add(o.x, o.a, o.b, o.ab_dtype, copy ? o.xb : nullptr, o.act_dtype, M, o.size, st), "residual_add")) return rc;
    if (int rc = product(ex, s, copy ? o.xb : (const void*)o.x, o.size, o.act_dtype, o.w_gate, o.size, o.w_dtype, o.g, o.dim, o.act_dtype, M, o.dim,
                         o.size, st))
        return rc;
    if (int rc = ex.launched(gate(o.g, o.dim, o.act_dtype, s.token_ids, o.table, o.table_dtype, o.ld_table, o.offset, o.vocab, o.g, o.dim, M,
                                  o.dim, st), "gelu_gather_mul"))
        return rc;
    if (int rc = product(ex, s, o.g, o.dim, o.act_dtype, o.w_proj, o.dim, o.w_dtype, o.y, o.size, LLME_DT_F32, M, o.size, o.dim, st)) return rc;
    return ex.launched(norm(o.x, o.y, o.gain, o.gain_dtype, M, o.size, o.eps, st), "rmsnorm_add");
}

int op_postnorm(LlmeExecutor& ex, const LlmePostNormOp& o, const LlmeStep& s, cudaStream_t st) {
    auto* f = (PostNormFn)ex.find("postnorm");
    if (!f) return ex.fail("no postnorm kernel is registered");
    return ex.launched(f(o.x, o.y, o.y_dtype, o.gain, o.gain_dtype, o.copy, o.copy_dtype, s.num_tokens, o.size, o.eps, o.accumulate, st), "postnorm");
}

int op_window_attention(LlmeExecutor& ex, const LlmeWindowAttentionOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    if (o.group < 0 || o.group >= s.num_groups) return ex.fail("window attention: the step has no cache group %d", o.group);
    const LlmeStepGroup& g = s.groups[o.group];
    auto* post = (WindowPostFn)ex.find("window_post");
    if (!post) return ex.fail("no window_post kernel is registered");
    LlmeWindowPostArgs p = {};
    p.q_in = o.q_in; p.k_in = o.k_in; p.v_in = o.v_in; p.q_stride = o.q_stride; p.k_stride = o.k_stride; p.v_stride = o.v_stride;
    p.q_gain = o.q_gain; p.k_gain = o.k_gain; p.eps = o.eps; p.inv_freq = o.inv_freq; p.rot_dims = o.rot_dims; p.amplitude = o.amplitude;
    p.positions = s.positions; p.q_out = o.q; p.cache = o.cache; p.slot_mapping = g.slot_mapping;
    p.tokens = s.num_tokens; p.nh = o.nh; p.nkv = o.nkv; p.dk = o.dk; p.dv = o.dv; p.page_size = g.page_size;
    p.q_bias = o.q_bias; p.k_bias = o.k_bias; p.v_bias = o.v_bias; p.head_norm = o.head_norm;
    p.interleaved = o.interleaved; p.in_f32 = o.in_f32;
    if (int rc = ex.launched(post(&p, o.dtype, st), "window_post")) return rc;
    // bfloat16 with sizes the tensor-core kernel is built for: prompt portions in one launch, single tokens in another
    auto* tc = (WindowAttnTcFn)ex.find("window_attention_tc/" + std::to_string(o.dk) + "x" + std::to_string(o.dv));
    if (tc && o.dtype == LLME_DT_BF16 && ex.choice("attention") == "fast") {
        LlmeWindowFastArgs f = {};
        f.q = o.q; f.cache = o.cache; f.out = o.out; f.sink = o.sink; f.cu_q_lens = s.cu_q_lens; f.ctx_lens = s.ctx_lens;
        f.table_rows = s.state_slots; f.block_tables = g.block_tables; f.max_blocks = g.max_blocks; f.nh = o.nh; f.nkv = o.nkv;
        f.page_size = g.page_size; f.window = o.window; f.keep_first = o.keep_first; f.scale = o.scale; f.softcap = o.softcap;
        if (s.num_portion > 0) {
            f.rows = s.portion_rows; f.n_rows = s.num_portion;
            if (int rc = ex.launched(tc(&f, s.max_portion_len, 0, st), "window_attention_tc")) return rc;
        }
        if (s.num_decode > 0) {
            f.rows = s.decode_rows; f.n_rows = s.num_decode;
            // key ranges: enough blocks for two an SM, no range shorter than two chunks of 64 keys, at most 8
            long long keys = s.max_decode_ctx;
            if (o.window > 0 && keys > (long long)o.window + o.keep_first) keys = (long long)o.window + o.keep_first;
            const long long chunks = keys / 64 + 1, units = (long long)s.num_decode * o.nkv;
            long long splits = (2LL * ex.sms + units - 1) / units;
            if (splits > chunks / 2) splits = chunks / 2;
            if (splits > 8) splits = 8;
            if (splits < 2 || o.nh / o.nkv > 64 || !o.scratch || (long long)s.num_decode * o.nh * splits * (o.dv + 2) > o.scratch_floats) splits = 1;
            f.splits = (int)splits; f.scratch = o.scratch;
            if (int rc = ex.launched(tc(&f, 1, s.max_decode_ctx, st), "window_attention_tc")) return rc;
            if (splits > 1) ++ex.launches;
        }
        return 0;
    }
    auto* plain = (WindowAttnPlainFn)ex.find("window_attention_plain");
    if (!plain) return ex.fail("no window attention kernel is registered");
    LlmeWindowAttnArgs a = {o.q, o.cache, o.out, o.sink, s.positions, s.token_request, g.block_tables, g.max_blocks, s.num_tokens,
                            o.nh, o.nkv, o.dk, o.dv, g.page_size, o.window, o.keep_first, o.scale, o.softcap};
    return ex.launched(plain(&a, o.dtype, st), "window_attention_plain");
}

int op_short_conv(LlmeExecutor& ex, const LlmeShortConvOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    auto* f = (ShortConvFn)ex.find("short_conv");
    if (!f) return ex.fail("no short_conv kernel is registered");
    LlmeShortConvArgs a = {o.x, o.ldx, o.x_dtype, o.w, o.bias, o.state, o.state_stride, o.out, o.ldo, s.cu_q_lens, s.state_slots,
                           s.num_tokens, s.num_requests, o.channels, o.taps, o.act};
    if (int rc = ex.launched(f(&a, 0, st), "short_conv")) return rc;
    if (o.taps <= 1) return 0;
    return ex.launched(f(&a, 1, st), "short_conv");     // after the outputs, which read the state: it takes the step's last inputs
}

int op_rotate(LlmeExecutor& ex, const LlmeRotateOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    auto* f = (RotateFn)ex.find("rotate");
    if (!f) return ex.fail("no rotate kernel is registered");
    LlmeRotateArgs a = {};
    for (int i = 0; i < 2; ++i) {
        a.x[i] = o.x[i]; a.ldx[i] = o.ldx[i]; a.out[i] = o.out[i]; a.ldo[i] = o.ldo[i]; a.heads[i] = o.heads[i]; a.scale[i] = o.scale[i];
    }
    a.dtype = o.dtype; a.dim = o.dim; a.rot_dims = o.rot_dims; a.inv_freq = o.inv_freq; a.positions = s.positions; a.tokens = s.num_tokens;
    return ex.launched(f(&a, st), "rotate");
}

int op_recurrence(LlmeExecutor& ex, const LlmeRecurrenceOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0 || s.num_requests <= 0) return 0;
    auto* f = (RecurrenceFn)ex.find("recurrence");
    if (!f) return ex.fail("no recurrence kernel is registered");
    LlmeRecurrenceArgs a = {o.q, o.k, o.ldq, o.ldk, o.qk_groups, o.v, o.ldv, o.v_dtype, o.gate, o.decay, o.dt, o.lddt, o.dt_dtype, o.dt_bias,
                            o.a_log, o.skip, o.state, o.state_stride, o.out, o.ldo, s.cu_q_lens, s.state_slots, s.num_requests, o.heads,
                            o.n, o.p, o.scratch, o.scratch_floats, s.num_tokens, s.max_portion_len > 1 ? s.max_portion_len : 1,
                            o.keep, o.take, o.ld_gates, o.unit_column};
    return ex.launched(f(&a, st), "recurrence");
}

int op_gated_norm(LlmeExecutor& ex, const LlmeGatedNormOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    auto* f = (GatedNormFn)ex.find("gated_norm");
    if (!f) return ex.fail("no gated_norm kernel is registered");
    LlmeGatedNormArgs a = {o.y, o.ldy, o.gate, o.ldg, o.weight, o.out, o.ldo, o.dtype, s.num_tokens, o.cols, o.group, o.gate_first, o.eps, o.scale,
                           o.gate_act, o.floor, o.ld_floor, o.den_eps};
    return ex.launched(f(&a, st), "gated_norm");
}

int op_row_norm(LlmeExecutor& ex, const LlmeRowNormOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    auto* f = (RowNormFn)ex.find("row_norm");
    if (!f) return ex.fail("no row_norm kernel is registered");
    return ex.launched(f(o.x, o.ldx, o.x_dtype, o.gain, o.gain_dtype, o.out, o.ldo, o.out_dtype, s.num_tokens, o.cols, o.eps, st), "row_norm");
}

int op_exp_gates(LlmeExecutor& ex, const LlmeExpGatesOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0 || s.num_requests <= 0) return 0;
    auto* f = (ExpGatesFn)ex.find("exp_gates");
    if (!f) return ex.fail("no exp_gates kernel is registered");
    LlmeExpGatesArgs a = {o.i_pre, o.f_pre, o.ld_pre, o.cap, o.state, o.state_stride, o.keep, o.take, o.floor, o.ld_out, s.cu_q_lens, s.state_slots,
                          s.num_requests, o.heads};
    return ex.launched(f(&a, s.max_portion_len > 1 ? s.max_portion_len : 1, st), "exp_gates");
}

int op_moe_route(LlmeExecutor& ex, const LlmeMoeRouteOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    auto* f = (MoeRouteFn)ex.find("moe_route");
    if (!f) return ex.fail("no moe_route kernel is registered");
    LlmeMoeRouteArgs a = {o.logits, o.ld, s.num_tokens, o.num_experts, o.top_k, o.scale, o.experts, o.weights, o.offsets, o.order, o.counts, o.mode};
    const int rc = ex.launched(f(&a, st), "moe_route");
    ++ex.launches;                                          // routing and ordering are two kernels
    return rc;
}

int op_grouped_linear(LlmeExecutor& ex, const LlmeGroupedLinearOp& o, const LlmeStep& s, cudaStream_t st) {
    if (s.num_tokens <= 0) return 0;
    LlmeGroupedArgs a = {o.x, o.ldx, o.w, o.ldw, o.w_expert, o.out, o.ldo, o.offsets, o.order, s.num_tokens * o.top_k, o.num_experts,
                         o.top_k, o.n, o.k, o.gather, o.scatter, o.act};
    // bfloat16 operands in whole 16-byte pieces: the tensor-core form (the activation in its epilogue)
    auto* tc = (GroupedFn)ex.find("grouped_linear_tc");
    if (tc && o.x_dtype == LLME_DT_BF16 && o.w_dtype == LLME_DT_BF16 && ex.choice("linear") != "plain" && o.k % 8 == 0 && o.ldx % 8 == 0 &&
        o.ldw % 8 == 0 && o.w_expert % 8 == 0 && aligned16(o.x, o.w))
        return ex.launched(tc(&a, o.x_dtype, o.w_dtype, o.out_dtype, st), "grouped_linear_tc");
    auto* f = (GroupedFn)ex.find("grouped_linear");
    if (!f) return ex.fail("no grouped_linear kernel is registered");
    return ex.launched(f(&a, o.x_dtype, o.w_dtype, o.out_dtype, st), "grouped_linear");
}

int op_moe_combine(LlmeExecutor& ex, const LlmeMoeCombineOp& o, const LlmeStep& s, cudaStream_t st) {
    if (o.base_gate) {
        auto* g = (MoeCombineGatedFn)ex.find("moe_combine_gated");
        if (!g) return ex.fail("no moe_combine kernel with a gate on the shared part is registered");
        return ex.launched(g(o.y, o.ldy, o.weights, o.base, o.out, s.num_tokens, o.top_k, o.size, o.base_gate, o.ld_gate, st), "moe_combine");
    }
    auto* f = (MoeCombineFn)ex.find("moe_combine");
    if (!f) return ex.fail("no moe_combine kernel is registered");
    return ex.launched(f(o.y, o.ldy, o.weights, o.base, o.out, s.num_tokens, o.top_k, o.size, st), "moe_combine");
}

const std::map<std::string, std::vector<std::string>>& variants() {
    static const std::map<std::string, std::vector<std::string>> v = {
        {"linear", {"auto", "tcgen05", "cublas", "plain"}},
        {"linear.decode", {"auto", "skinny", "cublas"}},
        {"linear_swiglu", {"fused", "unfused"}},
        {"attention", {"fast", "plain"}},
        {"attention.portion", {"tcgen05", "mma"}},
        {"attention.decode", {"fused", "split"}},
    };
    return v;
}

}  // namespace

// (every library of this package has this symbol; the executor's own messages belong to an executor: llme_executor_error)
LLME_EXPORT const char* llme_last_error() { return ""; }

LLME_EXPORT LlmeExecutor* llme_executor_create(int device) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
        cudaGetLastError();
        return nullptr;
    }
    auto* ex = new LlmeExecutor();
    ex->device = device;
    ex->sms = sms;
    for (auto& kv : variants()) ex->chosen[kv.first] = kv.second[0];
    return ex;
}

LLME_EXPORT void llme_executor_destroy(LlmeExecutor* ex) {
    if (!ex) return;
    if (ex->own_handle) ex->blas.destroy(ex->own_handle);
    if (ex->own_workspace) cudaFree(ex->own_workspace);
    delete ex;
}

LLME_EXPORT int llme_executor_register(LlmeExecutor* ex, const char* name, void* entry_point) {
    if (!name || !entry_point) return ex->fail("register: a name and an entry point are needed");
    ex->entry[name] = entry_point;
    return 0;
}

LLME_EXPORT int llme_executor_choose(LlmeExecutor* ex, const char* op, const char* variant) {
    const std::string o = op ? op : "", v = variant ? variant : "";
    if (o == "*") {
        if (v != "fast" && v != "plain") return ex->fail("choose: all operations at once take 'fast' or 'plain', got '%s'", v.c_str());
        for (auto& kv : variants()) ex->chosen[kv.first] = kv.second[0];
        if (v == "plain") {
            ex->chosen["linear"] = "plain";
            ex->chosen["linear_swiglu"] = "unfused";
            ex->chosen["attention"] = "plain";
        }
        return 0;
    }
    auto it = variants().find(o);
    if (it == variants().end()) {
        std::string known;
        for (auto& kv : variants()) known += (known.empty() ? "" : ", ") + kv.first;
        return ex->fail("choose: no operation '%s'; known: %s", o.c_str(), known.c_str());
    }
    for (auto& k : it->second)
        if (k == v) {
            ex->chosen[o] = v;
            return 0;
        }
    std::string known;
    for (auto& k : it->second) known += (known.empty() ? "" : ", ") + k;
    return ex->fail("choose: operation '%s' has no variant '%s'; it has: %s", o.c_str(), v.c_str(), known.c_str());
}

LLME_EXPORT const char* llme_executor_chosen(LlmeExecutor* ex, const char* op) {
    auto it = ex->chosen.find(op ? op : "");
    return it == ex->chosen.end() ? "" : it->second.c_str();
}

LLME_EXPORT const char* llme_executor_error(LlmeExecutor* ex) { return ex->error.c_str(); }
LLME_EXPORT long long llme_executor_launches(LlmeExecutor* ex) { return ex->launches; }

LLME_EXPORT int llme_decode_splits(LlmeExecutor* ex, int requests, int nh, int nkv, int hd, int window, int max_ctx) {
    if (requests <= 0 || nh <= 0 || nkv <= 0 || nh % nkv) return 1;
    return decode_splits(*ex, requests, nh, nkv, hd, window, max_ctx);
}

LLME_EXPORT long long llme_attention_scratch_floats(LlmeExecutor* ex, int max_requests, int nh, int nkv, int hd) {
    if (max_requests <= 0 || nh <= 0 || nkv <= 0 || nh % nkv) return 0;
    long long most = 0;
    for (int n = 1; n <= max_requests; ++n) {
        const int splits = decode_splits(*ex, n, nh, nkv, hd, 0, 1LL << 30);
        const long long need = splits <= 1 ? 0 : 65536 + (long long)n * nh * splits * (hd + 2);
        if (need > most) most = need;
    }
    return most;
}

LLME_EXPORT long long llme_latent_scratch_floats(LlmeExecutor* ex, int nh, int rank) {
    // requests x splits never exceeds the number of SMs (latent_splits)
    return nh <= 0 || rank <= 0 ? 0 : (long long)ex->sms * nh * (rank + 2);
}

LLME_EXPORT LlmePlan* llme_plan_create(LlmeExecutor* ex) {
    auto* p = new LlmePlan();
    p->ex = ex;
    return p;
}
LLME_EXPORT void llme_plan_destroy(LlmePlan* p) { delete p; }
LLME_EXPORT int llme_plan_size(LlmePlan* p) { return (int)p->records.size(); }

LLME_EXPORT int llme_plan_add(LlmePlan* p, int kind, const void* record, size_t bytes) {
    const size_t want = record_size(kind);
    if (!want) return p->ex->fail("plan: unknown record kind %d", kind);
    if (!record || bytes != want) return p->ex->fail("plan: a %s record has %zu bytes, got %zu", kind_name(kind), want, bytes);
    LlmePlan::Record r;
    r.kind = kind;
    r.bytes.assign((const unsigned char*)record, (const unsigned char*)record + bytes);
    p->records.push_back(std::move(r));
    return (int)p->records.size() - 1;
}

LLME_EXPORT int llme_plan_run(LlmePlan* p, const LlmeStep* step, int first, int count, cudaStream_t stream) {
    LlmeExecutor& ex = *p->ex;
    if (!step) return ex.fail("run: no step");
    const int n = (int)p->records.size();
    if (first < 0 || first > n) return ex.fail("run: record %d of %d", first, n);
    const int last = count < 0 || first + count > n ? n : first + count;
    const LlmeStep& s = *step;
    for (int i = first; i < last; ++i) {
        const LlmePlan::Record& r = p->records[i];
        const void* b = r.bytes.data();
        int rc = 0;
        switch (r.kind) {
            case LLME_OP_EMBEDDING: rc = op_embedding(ex, *(const LlmeEmbeddingOp*)b, s, stream); break;
            case LLME_OP_RMSNORM: rc = op_rmsnorm(ex, *(const LlmeRmsNormOp*)b, s, stream); break;
            case LLME_OP_LINEAR: rc = op_linear(ex, *(const LlmeLinearOp*)b, s, stream); break;
            case LLME_OP_LINEAR_SWIGLU: rc = op_linear_swiglu(ex, *(const LlmeLinearSwigluOp*)b, s, stream); break;
            case LLME_OP_QKV_POST: rc = op_qkv_post(ex, *(const LlmeQkvPostOp*)b, s, stream); break;
            case LLME_OP_ATTEND: rc = op_attend(ex, *(const LlmeAttendOp*)b, s, stream); break;
            case LLME_OP_ATTENTION: rc = op_attention(ex, *(const LlmeAttentionOp*)b, s, stream); break;
            case LLME_OP_LINEAR_ACT: rc = op_linear_act(ex, *(const LlmeLinearActOp*)b, s, stream); break;
            case LLME_OP_POINTWISE: rc = op_pointwise(ex, *(const LlmePointwiseOp*)b, s, stream); break;
            case LLME_OP_BATCHED_LINEAR: rc = op_batched_linear(ex, *(const LlmeBatchedLinearOp*)b, s, stream); break;
            case LLME_OP_RESIDUAL_ADD: rc = op_residual_add(ex, *(const LlmeResidualAddOp*)b, s, stream); break;
            case LLME_OP_LATENT_ATTENTION: rc = op_latent_attention(ex, *(const LlmeLatentAttentionOp*)b, s, stream); break;
            case LLME_OP_TOKEN_SIDE: rc = op_token_side(ex, *(const LlmeTokenSideOp*)b, s, stream); break;
            case LLME_OP_POSTNORM: rc = op_postnorm(ex, *(const LlmePostNormOp*)b, s, stream); break;
            case LLME_OP_WINDOW_ATTENTION: rc = op_window_attention(ex, *(const LlmeWindowAttentionOp*)b, s, stream); break;
            case LLME_OP_MOE_ROUTE: rc = op_moe_route(ex, *(const LlmeMoeRouteOp*)b, s, stream); break;
            case LLME_OP_GROUPED_LINEAR: rc = op_grouped_linear(ex, *(const LlmeGroupedLinearOp*)b, s, stream); break;
            case LLME_OP_MOE_COMBINE: rc = op_moe_combine(ex, *(const LlmeMoeCombineOp*)b, s, stream); break;
            case LLME_OP_SHORT_CONV: rc = op_short_conv(ex, *(const LlmeShortConvOp*)b, s, stream); break;
            case LLME_OP_ROTATE: rc = op_rotate(ex, *(const LlmeRotateOp*)b, s, stream); break;
            case LLME_OP_RECURRENCE: rc = op_recurrence(ex, *(const LlmeRecurrenceOp*)b, s, stream); break;
            case LLME_OP_GATED_NORM: rc = op_gated_norm(ex, *(const LlmeGatedNormOp*)b, s, stream); break;
            case LLME_OP_ROW_NORM: rc = op_row_norm(ex, *(const LlmeRowNormOp*)b, s, stream); break;
            case LLME_OP_EXP_GATES: rc = op_exp_gates(ex, *(const LlmeExpGatesOp*)b, s, stream); break;
            case LLME_OP_CALL: {
                const LlmeCallOp& c = *(const LlmeCallOp*)b;
                rc = c.fn ? c.fn(c.user, step, stream) : 0;
                if (rc) ex.error = "a called part reported an error";
                break;
            }
        }
        if (rc) {
            ex.error = "record " + std::to_string(i) + " (" + kind_name(r.kind) + "): " + ex.error;
            return rc;
        }
    }
    return 0;
}

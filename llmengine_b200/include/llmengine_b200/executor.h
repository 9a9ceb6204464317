/* llmengine_b200: the step executor.
 *
 * A model is flattened once, when it is loaded, into a *plan*: a list of operation records (embedding, norm,
 * matrix product, attention, ...), each holding the device pointers of its weights and of its places in the
 * step's workspace.  `llme_plan_run` then walks that list for one step: a batch of (request, its next tokens)
 * that may mix prompt portions with single decoded tokens, described by an `LlmeStep`.  The walk is native code:
 * per operation it decides which kernel serves the step's shape (the kernel registry below) and launches it on
 * the given stream; nothing is allocated and the host never waits for the device.
 *
 * The reference walks a graph of nodes and looks every kernel up per node and run
 * (src/runtime/executor.cpp:112-142, include/minillm/runtime/kernel_registry.h:18-35); the plan is the same
 * idea with the lookup done once and the shapes left open until the step.
 *
 * Kernels are not linked into this library.  Whoever loaded the kernel libraries registers their entry points
 * by name (`llme_executor_register`); an operation with several implementations (this package's tcgen05 or
 * mma.sync kernels, the plain 32-bit twins, the library product) is switched per operation with
 * `llme_executor_choose`, so that any fast kernel can be exchanged for its plain twin inside the whole model.
 *
 * An operation this library does not know is a `LLME_OP_CALL` record: a function pointer with a user value,
 * called in its turn with the step and the stream.  Parts written outside this package (also in Python) run
 * through it, and a new kernel family needs no change here.
 */
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLME_MAX_GROUPS 32   /* every distinct (window, kept first positions) among a model's layers is a group */

enum { LLME_DT_F32 = 0, LLME_DT_BF16 = 1 };

/* One cache group (layers whose caches grow and shrink together) as a step sees it. */
typedef struct LlmeStepGroup {
    const int* block_tables;   /* device [slots, max_blocks]; -1 where no page is held */
    const int* slot_mapping;   /* device [T]: page * page_size + place in page of each token; < 0 = not stored */
    int max_blocks, page_size, window;
} LlmeStepGroup;

/* One step.  Pointers are device memory and stay the same from step to step (a captured step is replayed with
 * new contents behind them); the counts are host values. */
typedef struct LlmeStep {
    int num_tokens, num_requests, num_logit_rows, num_decode, num_portion;
    int max_portion_len;       /* longest prompt portion of the step (requests with more than one token) */
    int max_decode_ctx;        /* longest context among the requests with exactly one token; for a step that is
                                  captured for replay: the longest context a replay may meet */
    const int* token_ids;      /* [T] */
    const int* positions;      /* [T] absolute position of each token in its request */
    const int* token_request;  /* [T] block-table row (state slot) of the token's request */
    const int* cu_q_lens;      /* [R+1] */
    const int* ctx_lens;       /* [R] cached length of each request after this step */
    const int* state_slots;    /* [R] */
    const int* first_portion;  /* [R] */
    const int* logit_rows;     /* [NL] token rows whose logits are wanted */
    const int* decode_rows;    /* [ND] batch rows of the requests with exactly one token */
    const int* portion_rows;   /* [NP] the others */
    float* logits;             /* [NL, vocab] output of the step */
    void* blas;                /* cublasHandle_t bound to `stream` by the caller, or NULL: the executor's own */
    int num_groups;
    LlmeStepGroup groups[LLME_MAX_GROUPS];
} LlmeStep;

typedef int (*LlmeCallFn)(void* user, const LlmeStep* step, cudaStream_t stream);

enum LlmeOpKind {
    LLME_OP_EMBEDDING = 1, LLME_OP_RMSNORM, LLME_OP_LINEAR, LLME_OP_LINEAR_SWIGLU, LLME_OP_QKV_POST, LLME_OP_ATTEND,
    LLME_OP_ATTENTION, LLME_OP_CALL, LLME_OP_LINEAR_ACT, LLME_OP_POINTWISE, LLME_OP_BATCHED_LINEAR, LLME_OP_RESIDUAL_ADD,
    LLME_OP_LATENT_ATTENTION, LLME_OP_TOKEN_SIDE, LLME_OP_POSTNORM, LLME_OP_WINDOW_ATTENTION, LLME_OP_MOE_ROUTE,
    LLME_OP_GROUPED_LINEAR, LLME_OP_MOE_COMBINE, LLME_OP_SHORT_CONV, LLME_OP_ROTATE, LLME_OP_RECURRENCE, LLME_OP_GATED_NORM,
    LLME_OP_ROW_NORM, LLME_OP_EXP_GATES
};

enum { LLME_ACT_XIELU = 1 };
/* activations of a (gate, up) pair: g sigmoid(g) u; with p0 = limit, p1 = slope: g' = min(g, limit),
 * u' = clamp(u, -limit, limit), g' sigmoid(slope g') (u' + 1) */
enum { LLME_GATE_SILU = 0, LLME_GATE_CLAMPED_SWISH = 1, LLME_GATE_GELU_TANH = 2 };   /* 2: gelu(g) u, the tanh form of gelu */
enum { LLME_POINTWISE_SIGMOID_MUL = 1 };

enum { LLME_ROWS_TOKENS = 0, LLME_ROWS_LOGITS = 1 };

typedef struct LlmeEmbeddingOp {
    const void* table; int table_dtype, vocab, hidden;
    float* out;                /* [T, hidden] */
    float scale;               /* every row times this constant, in 32-bit (1: none) */
} LlmeEmbeddingOp;

typedef struct LlmeRmsNormOp {
    float* x;                  /* [T, size] the residual stream, updated in place when delta is given */
    const void* delta; int delta_dtype;
    const void* gain; int gain_dtype;
    void* out; int out_dtype;
    int size; float eps;
    int rows;                  /* LLME_ROWS_TOKENS: every row; LLME_ROWS_LOGITS: the step's logit rows only */
    const void* gain2; void* out2;   /* a second gain and place for the same normed rows (the types of the first), or NULL */
} LlmeRmsNormOp;

typedef struct LlmeLinearOp {
    const void* x; long long ldx; int x_dtype;
    const void* w; long long ldw; int w_dtype;
    void* out; long long ldo; int out_dtype;   /* out NULL: the step's logits, row stride n */
    int n, k;
    int rows;                  /* LLME_ROWS_TOKENS or LLME_ROWS_LOGITS */
    const float* bias;         /* [n] added to every row of the product, or NULL */
} LlmeLinearOp;

typedef struct LlmeLinearSwigluOp {
    const void* x; long long ldx; int dtype;
    const void* w_gate_up; long long ldw;      /* [2 * inter, k]: gate rows, then up rows */
    void* gate_up;             /* [T, 2 * inter] workspace for the unfused form */
    void* out; long long ldo;  /* [T, inter] */
    int inter, k;
    int act; float p0, p1;     /* LLME_GATE_* and its constants */
    const float* bias;         /* [2 * inter] biases of the gate and up rows, added before the activation, or NULL */
} LlmeLinearSwigluOp;

/* QK norm, rotation and cache write as a step of its own (the parts of it that are given). */
typedef struct LlmeQkvPostOp {
    const void* q_in; const void* k_in; const void* v_in; long long q_stride, k_stride, v_stride; int in_dtype;
    const void* q_gain; const void* k_gain; int gain_dtype; float eps;
    const float* cos_sin; int max_positions;
    void* q_out; void* k_out; int out_dtype;
    void* cache; int group;    /* cache NULL: nothing is stored */
    int nh, nkv, hd;
} LlmeQkvPostOp;

/* Attention of every token of the step over its request's cache, queries finished. */
typedef struct LlmeAttendOp {
    const void* q; void* out; int dtype;
    const void* cache; long long cache_rows;   /* pages * 2 * nkv * page_size */
    int group, nh, nkv, hd, window; float scale;
    float* scratch; long long scratch_floats;
} LlmeAttendOp;

/* The mixer's middle in one record: raw q|k|v projections in, attention output out.  A step of single new tokens
 * goes to the decode kernel that norms, rotates and stores by itself; any other step to QKV_POST then ATTEND. */
typedef struct LlmeAttentionOp {
    LlmeQkvPostOp post;        /* q_out is the finished-queries workspace */
    LlmeAttendOp attend;
    const void* qkv; long long qkv_stride;
    int rotary;                /* 1: cos_sin table; 0: no position encoding at all */
} LlmeAttentionOp;

typedef struct LlmeCallOp { LlmeCallFn fn; void* user; } LlmeCallOp;

/* out = act(x w^T).  LLME_ACT_XIELU with p0 = a_pos, p1 = a_neg: z > 0: a_pos z^2 + z/2, else a_neg (exp(z) - 1 - z) + z/2. */
typedef struct LlmeLinearActOp {
    LlmeLinearOp product;      /* its `out` is the workspace [T, n] of the form that runs product and activation apart */
    void* out; long long ldo;  /* [T, n], the type of x */
    int act; float p0, p1;
} LlmeLinearActOp;

/* Elementwise over the step's rows.  LLME_POINTWISE_SIGMOID_MUL: out = a * sigmoid(b) * scale; with group > 1, b has one
 * value for every `group` neighbouring columns of a. */
typedef struct LlmePointwiseOp {
    int what, dtype, cols;
    const void* a; long long lda;
    const void* b; long long ldb;
    void* out; long long ldo;
    float scale;
    int group;
} LlmePointwiseOp;

/* out[t, b, :] = w[b] x[t, b, :] for b < batch: one small matrix per member (a head). */
typedef struct LlmeBatchedLinearOp {
    const void* x; long long ldx, x_member; int x_dtype;     /* row stride, stride between members */
    const void* w; long long ldw, w_member; int w_dtype;     /* [batch, n, k] */
    void* out; long long ldo, out_member; int out_dtype;
    int batch, n, k;
} LlmeBatchedLinearOp;

/* x += a (+ b): contributions that no following norm adds; each times its vector [size] first, where it has one. */
typedef struct LlmeResidualAddOp {
    float* x; const void* a; const void* b; int dtype; int size;
    const float* a_scale; const float* b_scale;
} LlmeResidualAddOp;

/* Attention over cached latent rows [c | rotated key part] shared by all heads (csrc/attention_latent.cu), from the
 * raw down-projection: norm of c, rotation of the key part and of the heads' rotated query parts, cache write, attention. */
typedef struct LlmeLatentAttentionOp {
    const void* kv_in; long long kv_stride;                   /* [T, rank + rot] */
    const void* q_rot; long long q_rot_stride, q_rot_head_stride;   /* [T, nh, rot] view, or NULL */
    const void* c_gain; int gain_dtype; float eps;
    const float* inv_freq; int rot_dims;
    void* q; void* out; int dtype;                            /* q [T, nh, rank + rot]; out [T, nh, rank] */
    void* cache; long long cache_rows; int group;
    int nh, rank, rot; float scale;
    const float* sink;                                        /* [nh] or NULL */
    float* scratch; long long scratch_floats;
    int window;                                               /* W > 0: query i sees key j only if i - j < W */
    int interleaved;                                          /* 1: the rotation pairs coordinate 2i with 2i + 1 */
} LlmeLatentAttentionOp;

/* x += a (+ b); e = table[token][offset .. offset + dim); g = gelu_tanh(w_gate x) * e; y = w_proj g;
 * x += y / sqrt(mean(y^2) + eps) * gain. */
typedef struct LlmeTokenSideOp {
    float* x; const void* a; const void* b; int ab_dtype; int size;
    const void* table; int table_dtype; long long ld_table; int offset, dim, vocab;
    const void* w_gate; const void* w_proj; int w_dtype;      /* [dim, size], [size, dim] */
    const void* gain; int gain_dtype; float eps;
    void* xb; void* g; int act_dtype; float* y;               /* workspace: [T, size], [T, dim], [T, size] */
} LlmeTokenSideOp;

/* The norm on a sublayer's output: x += y / sqrt(mean(y^2) + eps) * gain (accumulate 0: x = ...; y may be x), and the
 * new x written to `copy` in its type; y NULL: only the copy. */
typedef struct LlmePostNormOp {
    float* x; const void* y; int y_dtype;
    const void* gain; int gain_dtype; float eps;
    void* copy; int copy_dtype;
    int size, accumulate;
} LlmePostNormOp;

/* Grouped-query attention with keys dk and values dv wide, from the raw projections: norm of q and k over the whole
 * projection, rotation of the first rot_dims coordinates of every head, cache write, then attention in which query i
 * sees key j if j <= i and (i - j < window or j < keep_first), with an optional sink per head in the denominator
 * (csrc/attention_window.cu; a cache page holds [nkv][page][dk] keys, then [nkv][page][dv] values). */
typedef struct LlmeWindowAttentionOp {
    const void* q_in; const void* k_in; const void* v_in; long long q_stride, k_stride, v_stride; int dtype;
    const float* q_gain; const float* k_gain; float eps;
    const float* inv_freq; int rot_dims; float amplitude;
    void* q; void* out;                                       /* [T, nh dk] workspace; [T, nh dv] */
    void* cache; int group;
    int nh, nkv, dk, dv, window, keep_first; float scale;
    const float* sink;
    float* scratch; long long scratch_floats;                /* for single tokens whose keys are cut into ranges, or NULL */
    /* options (off when zero): biases of the projections, added first; head_norm 1: every head is normed by itself and the
     * gains are [dk], shared by the heads.  v_in may be k_in itself: the values are then the keys as projected. */
    const float* q_bias; const float* k_bias; const float* v_bias; int head_norm;
    float softcap;                                           /* c > 0: a score s becomes c tanh(s / c) behind the scale */
    int interleaved;                                         /* 1: the rotation pairs coordinate 2i with 2i + 1 */
    int in_f32;                                              /* 1: q_in, k_in, v_in are 32-bit whatever `dtype` is (they come from a convolution) */
} LlmeWindowAttentionOp;

/* Routing of a mixture of experts: s = sigmoid(logits), the top_k largest, w_e = scale * s_e / (sum of the chosen s + 1e-20);
 * the (token, choice) pairs listed expert by expert (csrc/moe.cu). */
typedef struct LlmeMoeRouteOp {
    const float* logits; long long ld; int num_experts, top_k; float scale;
    int* experts; float* weights; int* offsets; int* order; int* counts;
    int mode;                  /* 0: as above; 1: the largest logits chosen, w_e = scale * softmax over the chosen logits alone */
} LlmeMoeRouteOp;

/* One product per expert over the pairs routed to it. */
typedef struct LlmeGroupedLinearOp {
    const void* x; long long ldx; int x_dtype;
    const void* w; long long ldw, w_expert; int w_dtype;      /* [E, n, k] */
    void* out; long long ldo; int out_dtype;
    void* mid; long long ld_mid;                              /* [pairs, n]: workspace of the unfused activation, or NULL */
    const int* offsets; const int* order;
    int num_experts, top_k, n, k, gather, scatter, act;       /* act 1: w[e] = [gate | up], out = silu(gate) * up */
} LlmeGroupedLinearOp;

/* out[t] = base[t] (times sigmoid(base_gate[t * ld_gate]) where base_gate is given) + sum_k weights[t, k] y[t top_k + k]. */
typedef struct LlmeMoeCombineOp {
    const float* y; long long ldy; const float* weights; const float* base; float* out; int top_k, size;
    const float* base_gate; long long ld_gate;
} LlmeMoeCombineOp;

/* Causal convolution per channel over each request's tokens, y_t = bias + sum_j w[:, K-1-j] x_(t-j), then silu (act 1);
 * the request's last K - 1 inputs live in its state slot ([K - 1, channels] 32-bit, zero when the request starts). */
typedef struct LlmeShortConvOp {
    const void* x; long long ldx; int x_dtype;
    const float* w; const float* bias;
    float* state; long long state_stride;
    float* out; long long ldo;
    int channels, taps, act;
} LlmeShortConvOp;

/* Rotation of the first rot_dims coordinates of every head of up to two tensors by the tokens' positions (rotate-half
 * pairs, angle position * inv_freq[i]), each then times a constant; results in 32-bit. */
typedef struct LlmeRotateOp {
    const void* x[2]; long long ldx[2]; float* out[2]; long long ldo[2]; int heads[2]; float scale[2];
    int dtype, dim, rot_dims;
    const float* inv_freq;
} LlmeRotateOp;

/* Linear recurrence with a matrix state per head and request: S_t = a_t S_(t-1) + s_t k_t v_t^T, y_t = S_t^T q_t + skip_h v_t
 * (csrc/recurrent.cu).  gate 0: a_t = decay[h], s_t = 1; gate 1: d = softplus(dt[t, h] + dt_bias[h]), a_t = exp(-exp(a_log[h]) d),
 * s_t = d.  State [heads, p, n] 32-bit per slot, zero when the request starts. */
typedef struct LlmeRecurrenceOp {
    const float* q; const float* k; long long ldq, ldk; int qk_groups;
    const void* v; long long ldv; int v_dtype;
    int gate;
    const float* decay;
    const void* dt; long long lddt; int dt_dtype; const float* dt_bias; const float* a_log;
    const float* skip;
    float* state; long long state_stride;
    float* out; long long ldo;
    int heads, n, p;
    float* scratch; long long scratch_floats;                /* lets long portions run in pieces side by side, or NULL */
    /* gate 2: a_t = keep[t, h], s_t = take[t, h] (32-bit, row stride ld_gates), made by an earlier record */
    const float* keep; const float* take; long long ld_gates;
    int unit_column;                                         /* 1: column p - 1 has no v behind it, its v_t is one; v is [T, heads (p - 1)] */
} LlmeRecurrenceOp;

/* RMS norm in groups of `group` columns with a silu gate: gate_first 1: u = y silu(g), out = u / rms(u) * weight; 0:
 * out = y / rms(y) * weight * silu(g); then times `scale`. */
typedef struct LlmeGatedNormOp {
    const float* y; long long ldy;
    const void* gate; long long ldg;
    const float* weight;
    void* out; long long ldo;
    int dtype, cols, group, gate_first;
    float eps, scale;
    int gate_act;                                            /* 0: silu(g); 1: sigmoid(g) */
    /* with `floor` [T, cols / group] every group of y is one value wider: the extra value d stands behind the group's own, and
     * the group is divided by max(|d|, floor) + den_eps before anything else */
    const float* floor; long long ld_floor; float den_eps;
} LlmeGatedNormOp;

/* out = x / sqrt(mean(x^2) + eps) * gain over the rows of x: a norm on (a column range of) a product. */
typedef struct LlmeRowNormOp {
    const void* x; long long ldx; int x_dtype;
    const void* gain; int gain_dtype;
    void* out; long long ldo; int out_dtype;
    int cols; float eps;
} LlmeRowNormOp;

/* The gates of a matrix memory with exponential gating, per request and head over the request's tokens (csrc/recurrent.cu):
 * a_t = cap tanh(i_pre / cap), b_t = logsigmoid(cap tanh(f_pre / cap)) (cap 0: uncapped), M_t = max(b_t + M_(t-1), a_t) with M in
 * the request's state slot ([heads] 32-bit, zero when the request starts); keep = exp(b_t + M_(t-1) - M_t), take = exp(a_t - M_t),
 * floor = exp(-M_t). */
typedef struct LlmeExpGatesOp {
    const float* i_pre; const float* f_pre; long long ld_pre;
    float cap;
    float* state; long long state_stride;
    float* keep; float* take; float* floor; long long ld_out;
    int heads;
} LlmeExpGatesOp;

typedef struct LlmeExecutor LlmeExecutor;
typedef struct LlmePlan LlmePlan;

LlmeExecutor* llme_executor_create(int device);
void llme_executor_destroy(LlmeExecutor*);
/* Entry points of the kernel libraries, by name: "embedding", "rmsnorm", "qkv_post", "swiglu", "gemm_f32",
 * "gemm_skinny", "gemm_skinny_swiglu", "gemm_tc", "gemm_tc_swiglu", "attention_plain", and per head size
 * "attention_portion/<hd>", "attention_decode/<hd>", "attention_decode_fused/<hd>", "attention_tc/<hd>"; "xielu",
 * "sigmoid_mul", "residual_add", "gelu_gather_mul", "rmsnorm_add", "latent_post", "gemm_f32_batched",
 * "latent_attention_plain", and per latent size "latent_attention_tc/<rank>", "latent_attention_tc_fits/<rank>";
 * "postnorm", "gated_act", "gemm_skinny_gated", "gemm_tc_gated", "window_post", "window_attention_plain", per pair of
 * key and value sizes "window_attention_tc/<dk>x<dv>", "moe_route", "grouped_linear", "grouped_linear_tc", "moe_combine";
 * "short_conv", "rotate", "recurrence", "gated_norm", "row_norm", "exp_gates", "sigmoid_mul_grouped", "residual_add_scaled",
 * "moe_combine_gated". */
int llme_executor_register(LlmeExecutor*, const char* name, void* entry_point);
/* Which implementation an operation takes.  Operations and their variants:
 *   "linear":            "auto" | "tcgen05" | "cublas" | "plain"   (bfloat16 products of 128 tokens or more / all)
 *   "linear.decode":     "auto" | "skinny" | "cublas"               (bfloat16 products of up to 16 tokens)
 *   "linear_swiglu":     "fused" | "unfused"
 *   "attention.portion": "tcgen05" | "mma" | "plain"
 *   "attention.decode":  "fused" | "split" | "plain"
 *   "*":                 "fast" | "plain"                           (all of the above at once)
 * Returns 0, or -1 for an unknown operation or variant. */
int llme_executor_choose(LlmeExecutor*, const char* op, const char* variant);
const char* llme_executor_chosen(LlmeExecutor*, const char* op);
const char* llme_executor_error(LlmeExecutor*);
long long llme_executor_launches(LlmeExecutor*);      /* kernels of this package launched so far */
/* Scratch floats an attention record needs for steps of up to `max_requests` single tokens. */
long long llme_attention_scratch_floats(LlmeExecutor*, int max_requests, int nh, int nkv, int hd);
/* Scratch floats a latent attention record needs for any step of single tokens. */
long long llme_latent_scratch_floats(LlmeExecutor*, int nh, int rank);
/* Blocks per (request, key/value head) that the decode attention would use. */
int llme_decode_splits(LlmeExecutor*, int requests, int nh, int nkv, int hd, int window, int max_ctx);

LlmePlan* llme_plan_create(LlmeExecutor*);
void llme_plan_destroy(LlmePlan*);
/* Appends a record (copied); `kind` says which of the structs above `record` is.  Returns its index, or -1. */
int llme_plan_add(LlmePlan*, int kind, const void* record, size_t bytes);
int llme_plan_size(LlmePlan*);
/* Runs records [first, first + count) (count < 0: to the end) for one step.  0, or the failing record's code;
 * `llme_executor_error` then names the record and the reason. */
int llme_plan_run(LlmePlan*, const LlmeStep* step, int first, int count, cudaStream_t stream);

#ifdef __cplusplus
}

#include <stdexcept>
#include <string>

namespace llmengine_b200 {

/* Thin C++ face of the functions above: owning handles, errors as exceptions. */
class Executor {
public:
    explicit Executor(int device = 0) : h_(llme_executor_create(device)) {
        if (!h_) throw std::runtime_error("llmengine_b200: cannot create an executor on this device");
    }
    ~Executor() { llme_executor_destroy(h_); }
    Executor(const Executor&) = delete;
    Executor& operator=(const Executor&) = delete;
    void register_kernel(const std::string& name, void* entry) {
        if (llme_executor_register(h_, name.c_str(), entry)) throw std::invalid_argument(error());
    }
    void choose(const std::string& op, const std::string& variant) {
        if (llme_executor_choose(h_, op.c_str(), variant.c_str())) throw std::invalid_argument(error());
    }
    std::string error() const { return llme_executor_error(h_); }
    LlmeExecutor* handle() const { return h_; }

private:
    LlmeExecutor* h_;
};

class Plan {
public:
    explicit Plan(Executor& ex) : ex_(ex), h_(llme_plan_create(ex.handle())) {}
    ~Plan() { llme_plan_destroy(h_); }
    Plan(const Plan&) = delete;
    Plan& operator=(const Plan&) = delete;
    int add(const LlmeEmbeddingOp& r) { return add(LLME_OP_EMBEDDING, &r, sizeof r); }
    int add(const LlmeRmsNormOp& r) { return add(LLME_OP_RMSNORM, &r, sizeof r); }
    int add(const LlmeLinearOp& r) { return add(LLME_OP_LINEAR, &r, sizeof r); }
    int add(const LlmeLinearSwigluOp& r) { return add(LLME_OP_LINEAR_SWIGLU, &r, sizeof r); }
    int add(const LlmeQkvPostOp& r) { return add(LLME_OP_QKV_POST, &r, sizeof r); }
    int add(const LlmeAttendOp& r) { return add(LLME_OP_ATTEND, &r, sizeof r); }
    int add(const LlmeAttentionOp& r) { return add(LLME_OP_ATTENTION, &r, sizeof r); }
    int add(const LlmeCallOp& r) { return add(LLME_OP_CALL, &r, sizeof r); }
    int add(const LlmeLinearActOp& r) { return add(LLME_OP_LINEAR_ACT, &r, sizeof r); }
    int add(const LlmePointwiseOp& r) { return add(LLME_OP_POINTWISE, &r, sizeof r); }
    int add(const LlmeBatchedLinearOp& r) { return add(LLME_OP_BATCHED_LINEAR, &r, sizeof r); }
    int add(const LlmeResidualAddOp& r) { return add(LLME_OP_RESIDUAL_ADD, &r, sizeof r); }
    int add(const LlmeLatentAttentionOp& r) { return add(LLME_OP_LATENT_ATTENTION, &r, sizeof r); }
    int add(const LlmeTokenSideOp& r) { return add(LLME_OP_TOKEN_SIDE, &r, sizeof r); }
    int add(const LlmePostNormOp& r) { return add(LLME_OP_POSTNORM, &r, sizeof r); }
    int add(const LlmeWindowAttentionOp& r) { return add(LLME_OP_WINDOW_ATTENTION, &r, sizeof r); }
    int add(const LlmeMoeRouteOp& r) { return add(LLME_OP_MOE_ROUTE, &r, sizeof r); }
    int add(const LlmeGroupedLinearOp& r) { return add(LLME_OP_GROUPED_LINEAR, &r, sizeof r); }
    int add(const LlmeMoeCombineOp& r) { return add(LLME_OP_MOE_COMBINE, &r, sizeof r); }
    int add(const LlmeShortConvOp& r) { return add(LLME_OP_SHORT_CONV, &r, sizeof r); }
    int add(const LlmeRotateOp& r) { return add(LLME_OP_ROTATE, &r, sizeof r); }
    int add(const LlmeRecurrenceOp& r) { return add(LLME_OP_RECURRENCE, &r, sizeof r); }
    int add(const LlmeGatedNormOp& r) { return add(LLME_OP_GATED_NORM, &r, sizeof r); }
    int add(const LlmeRowNormOp& r) { return add(LLME_OP_ROW_NORM, &r, sizeof r); }
    int add(const LlmeExpGatesOp& r) { return add(LLME_OP_EXP_GATES, &r, sizeof r); }
    /* One step through the whole plan; throws with the failing record's message. */
    void run(const LlmeStep& step, cudaStream_t stream) {
        if (llme_plan_run(h_, &step, 0, -1, stream)) throw std::runtime_error(ex_.error());
    }

private:
    int add(int kind, const void* r, size_t n) {
        const int i = llme_plan_add(h_, kind, r, n);
        if (i < 0) throw std::invalid_argument(ex_.error());
        return i;
    }
    Executor& ex_;
    LlmePlan* h_;
};

}  // namespace llmengine_b200
#endif

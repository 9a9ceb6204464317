/* Argument blocks of the kernel libraries' entry points, as plain C structs: what a caller outside the kernel
 * sources (the step executor, a binding) fills in.  Each kernel source keeps its own typed struct and asserts
 * that its layout equals the one here. */
#pragma once

typedef struct LlmeQkvArgs {
    const void* q_in; const void* k_in; const void* v_in;
    long long q_stride, k_stride, v_stride;      /* elements between consecutive tokens */
    const void* q_gain; const void* k_gain;       /* nullable: no norm */
    int gain_dtype;
    float eps;
    const float* cos_sin;                         /* nullable: no rotation; [max_pos, head_dim] = cos | sin */
    const int* positions;
    int max_positions;
    void* q_out; void* k_out;                     /* nullable; [T, nh*hd], [T, nkv*hd] */
    void* cache; const int* slot_mapping;         /* nullable */
    int tokens, nh, nkv, hd, page_size;
} LlmeQkvArgs;

typedef struct LlmeAttnArgs {
    const void* q; const void* cache; void* out;
    const int* positions; const int* token_request; const int* block_tables;
    int max_blocks;
    int tokens, nh, nkv, hd, page_size;
    int window;
    float scale;
} LlmeAttnArgs;

typedef struct LlmeFastAttnArgs {
    const void* q; const void* cache; void* out;
    const int* rows; const int* cu_q_lens; const int* ctx_lens; const int* table_rows; const int* block_tables;
    float* scratch;
    int max_blocks, n_rows, nh, nkv, page_size, window, splits;
    float scale;
} LlmeFastAttnArgs;

typedef struct LlmeFusedQkv {
    const void* qkv; long long stride;
    const void* q_gain; const void* k_gain; int gain_dtype; float eps;
    const float* cos_sin; int max_positions; int write_kv;
} LlmeFusedQkv;

typedef struct LlmeTcAttnArgs {
    void* out; const void* cache;
    const int* rows; const int* cu_q_lens; const int* ctx_lens; const int* table_rows; const int* block_tables;
    int max_blocks, n_rows, nh, nkv, page_size, window;
    float scale;
} LlmeTcAttnArgs;

/* Norm of the latent, rotation of the shared key part and of the heads' rotated query parts, cache write. */
typedef struct LlmeLatentPostArgs {
    const void* kv_in; long long kv_stride;       /* [T, rank + rot]: raw down-projection */
    const void* q_rot; long long q_rot_stride, q_rot_head_stride;   /* [T, nh, rot] view; nullable when rot == 0 */
    const void* c_gain; int gain_dtype; float eps;
    const float* inv_freq; int rot_dims;          /* rot_dims / 2 frequencies; the first rot_dims of rot are rotated */
    const int* positions;
    void* q;                                      /* [T, nh, rank + rot]: the last rot of every head are written */
    void* cache; const int* slot_mapping;         /* rows of rank + rot; slot < 0: not stored */
    int tokens, nh, rank, rot;
    int interleaved;                              /* 1: the rotation pairs coordinate 2i with 2i + 1, not i with i + rot_dims / 2 */
} LlmeLatentPostArgs;

/* Attention over cached latent rows [c | rotated key part], one row per token for all heads. */
typedef struct LlmeLatentAttnArgs {
    const void* q; const void* cache; void* out;  /* q [T, nh, rank + rot]; out [T, nh, rank] */
    const float* sink;                            /* [nh] or NULL */
    const int* positions; const int* token_request; const int* block_tables;
    int max_blocks, tokens, nh, rank, rot, page_size;
    float scale;
    int window;                                   /* W > 0: query i sees key j only if i - j < W */
} LlmeLatentAttnArgs;

/* Whole-projection norm, partial rotation and cache write for an attention whose keys and values differ in width
 * (csrc/attention_window.cu).  A cache page holds [nkv][page_size][dk] keys, then [nkv][page_size][dv] values. */
typedef struct LlmeWindowPostArgs {
    const void* q_in; const void* k_in; const void* v_in;   /* k_in / v_in NULL: nothing is stored */
    long long q_stride, k_stride, v_stride;
    const float* q_gain; const float* k_gain; float eps;     /* gains NULL: no norm; [nh * dk], [nkv * dk] */
    const float* inv_freq; int rot_dims; float amplitude;    /* inv_freq NULL: no rotation */
    const int* positions;
    void* q_out;                                             /* [T, nh * dk] */
    void* cache; const int* slot_mapping;
    int tokens, nh, nkv, dk, dv, page_size;
    /* options of other designs (all off when zero): biases of the three projections, added first (32-bit, [nh * dk],
     * [nkv * dk], [nkv * dv]); `head_norm` 1: every head is normed by itself and the gains are [dk], shared by the heads */
    const float* q_bias; const float* k_bias; const float* v_bias;
    int head_norm;
    int interleaved;                                         /* 1: the rotation pairs coordinate 2i with 2i + 1, not i with i + rot_dims / 2 */
    int in_f32;                                              /* 1: q_in, k_in and v_in are 32-bit whatever the type of q_out and the cache */
} LlmeWindowPostArgs;

/* Attention over such a cache: query i sees key j if j <= i and (i - j < window or j < keep_first). */
typedef struct LlmeWindowAttnArgs {
    const void* q; const void* cache; void* out;             /* q [T, nh * dk]; out [T, nh * dv] */
    const float* sink;                                       /* [nh] or NULL */
    const int* positions; const int* token_request; const int* block_tables;
    int max_blocks, tokens, nh, nkv, dk, dv, page_size, window, keep_first;
    float scale;
    float softcap;                                           /* c > 0: a score s becomes c tanh(s / c) behind the scale */
} LlmeWindowAttnArgs;

/* The same for the tensor-core kernel: the requests `rows` of the batch, each with its tokens
 * cu_q_lens[row] .. cu_q_lens[row + 1] that end at position ctx_lens[row] - 1. */
typedef struct LlmeWindowFastArgs {
    const void* q; const void* cache; void* out;
    const float* sink;
    const int* rows; const int* cu_q_lens; const int* ctx_lens; const int* table_rows; const int* block_tables;
    int max_blocks, n_rows, nh, nkv, page_size, window, keep_first;
    float scale;
    float* scratch; int splits;      /* single tokens: each request's keys cut into `splits` ranges whose parts meet in `scratch` */
    float softcap;                   /* c > 0: a score s becomes c tanh(s / c) behind the scale */
} LlmeWindowFastArgs;

/* Routing of a mixture of experts (csrc/moe.cu). */
typedef struct LlmeMoeRouteArgs {
    const float* logits; long long ld;                       /* [T, E] */
    int tokens, num_experts, top_k; float scale;
    int* experts; float* weights;                            /* [T, top_k] */
    int* offsets; int* order; int* counts;                   /* [E + 1], [T * top_k], [E] (zero between launches) */
    int mode;                                                /* 0: sigmoid scores normalised over the chosen; 1: softmax over the chosen logits */
} LlmeMoeRouteArgs;

/* One product per expert over the rows routed to it. */
typedef struct LlmeGroupedArgs {
    const void* x; long long ldx;
    const void* w; long long ldw, w_expert;                  /* [E, n, k] */
    void* out; long long ldo;
    const int* offsets; const int* order;
    int pairs, num_experts, top_k, n, k;                     /* pairs = tokens * top_k */
    int gather, scatter;                                     /* x row = order[r] / top_k; out row = order[r] */
    int act;                                                 /* 1: w[e] = [gate | up], the row written is silu(gate) * up, n / 2 wide */
} LlmeGroupedArgs;

/* Causal convolution per channel over the tokens of each request (csrc/recurrent.cu): y_t = bias + sum_j w[:, K-1-j] x_(t-j),
 * then the activation; the last K - 1 inputs of every request are carried in its state slot ([K - 1, channels], oldest first,
 * zero for a request that starts: the zeros before the start).  Two launches: `update` 0: the outputs of the step's tokens (the state is
 * read); 1: the state takes the step's last inputs (a launch of its own, after the first). */
typedef struct LlmeShortConvArgs {
    const void* x; long long ldx; int x_dtype;               /* [T, channels] (a column range of a product) */
    const float* w; const float* bias;                       /* [channels, taps]; [channels] or NULL */
    float* state; long long state_stride;                    /* slot s: state + s * state_stride */
    float* out; long long ldo;                               /* [T, channels] 32-bit */
    const int* cu_q_lens; const int* state_slots;
    int tokens, requests, channels, taps, act;               /* act 1: silu */
} LlmeShortConvArgs;

/* Rotation of the first rot_dims coordinates of every head (rotate-half pairs, angle position * inv_freq[i], 32-bit) of up
 * to two tensors, each times a constant afterwards; the results are 32-bit. */
typedef struct LlmeRotateArgs {
    const void* x[2]; long long ldx[2]; float* out[2]; long long ldo[2]; int heads[2]; float scale[2];   /* x[i] NULL: absent */
    int dtype, dim, rot_dims;
    const float* inv_freq; const int* positions;
    int tokens;
} LlmeRotateArgs;

/* A linear recurrence with a decaying matrix state per head and request (csrc/recurrent.cu):
 *   S_t = a_t S_(t-1) + s_t k_t v_t^T   (S is n x p),   y_t = S_t^T q_t + skip_h v_t.
 * gate 0: a_t = decay[h], s_t = 1.  gate 1: d = softplus(dt[t, h] + dt_bias[h]), a_t = exp(-exp(a_log[h]) d), s_t = d.
 * q and k come in `qk_groups` groups of n; head h reads group h / (heads / qk_groups).  The state lives in 32-bit in the
 * request's slot, one column of S after the other ([heads, p, n]), and goes from step to step. */
typedef struct LlmeRecurrenceArgs {
    const float* q; const float* k; long long ldq, ldk; int qk_groups;
    const void* v; long long ldv; int v_dtype;               /* [T, heads * p] */
    int gate;
    const float* decay;
    const void* dt; long long lddt; int dt_dtype; const float* dt_bias; const float* a_log;
    const float* skip;                                       /* [heads] or NULL */
    float* state; long long state_stride;                    /* slot s: [heads, p, n] at state + s * state_stride */
    float* out; long long ldo;                               /* [T, heads * p] 32-bit */
    const int* cu_q_lens; const int* state_slots;
    int requests, heads, n, p;
    float* scratch; long long scratch_floats;                /* room for the states of pieces of long requests, or NULL */
    int tokens, max_len;                                     /* of the step; the most tokens one request brings */
    /* gate 2: a_t = keep[t, h], s_t = take[t, h], 32-bit, made by an earlier kernel (row stride ld_gates) */
    const float* keep; const float* take; long long ld_gates;
    int unit_column;                                         /* 1: column p - 1 has no v behind it, its v_t is one; v is [T, heads * (p - 1)] */
} LlmeRecurrenceArgs;

/* RMS norm in groups of `group` columns with a gate (silu of a second tensor) before or after it:
 * gate_first 1: u = y silu(g), out = u / rms(u) * weight;  0: out = y / rms(y) * weight * silu(g); then times `scale`.
 * weight NULL: none.  y is 32-bit; g and out have `dtype`. */
typedef struct LlmeGatedNormArgs {
    const float* y; long long ldy;
    const void* gate; long long ldg;
    const float* weight;
    void* out; long long ldo;
    int dtype, tokens, cols, group, gate_first;
    float eps, scale;
    int gate_act;                                            /* 0: silu(g); 1: sigmoid(g) */
    /* with `floor` [T, cols / group] every group of y is one value wider than `group`: the extra value d stands behind the
     * group's own, and the group is divided by max(|d|, floor) + den_eps before anything else */
    const float* floor; long long ld_floor; float den_eps;
} LlmeGatedNormArgs;

/* The gates of a matrix memory with exponential gating (csrc/recurrent.cu), per request and head over the request's tokens:
 * a_t = cap tanh(i_pre / cap), b_t = logsigmoid(cap tanh(f_pre / cap)) (cap 0: uncapped), M_t = max(b_t + M_(t-1), a_t) with M
 * kept in the request's slot; keep = exp(b_t + M_(t-1) - M_t), take = exp(a_t - M_t), floor = exp(-M_t). */
typedef struct LlmeExpGatesArgs {
    const float* i_pre; const float* f_pre; long long ld_pre;   /* [T, heads] each */
    float cap;
    float* state; long long state_stride;                    /* slot s: [heads] at state + s * state_stride */
    float* keep; float* take; float* floor; long long ld_out;   /* [T, heads] each */
    const int* cu_q_lens; const int* state_slots;
    int requests, heads;
} LlmeExpGatesArgs;

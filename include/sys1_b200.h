/*
 * sys1_b200 - C ABI of the B200 (sm_100a) dense-projection / gated-delta-rule path.
 *
 * This is the boundary a sys1 maintainer binds from Rust (`extern "C"`) in place of the candle calls on the
 * model hot path. Every pointer below is a DEVICE pointer unless the name ends in `_host`; activations and
 * weights are bf16, row-major, rows at least 16-byte aligned (leading dimensions are multiples of 8 elements).
 * The caller owns every buffer it passes; the library keeps no copy of weights and allocates no activation.
 *
 * Conventions
 *   - every function returns 0 (S1_OK) or a negative S1_E* code; nothing throws or aborts across the boundary;
 *     `s1_last_error` gives the message of the last failing call on that context;
 *   - work is enqueued on the context's stream and is asynchronous; `s1_sync` joins it and reports errors the
 *     kernels recorded on the device (a wait inside a kernel that ran out of time, for instance);
 *   - one host thread per context at a time (the reference runs one `predict_batch` at a time,
 *     src/batching.rs:121); contexts on different GPUs are independent;
 *   - there is no CPU or library fallback: on a machine without an sm_100 GPU `s1_ctx_create` fails.
 */
#ifndef SYS1_B200_H_
#define SYS1_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct s1_ctx s1_ctx;

enum {
    S1_OK = 0,
    S1_EINVAL = -1,   /* bad argument: null pointer, shape or alignment the kernels cannot take */
    S1_ECUDA = -2,    /* a CUDA runtime / driver call failed */
    S1_EDEVICE = -3,  /* not an sm_100 device, or no device */
    S1_EKERNEL = -4,  /* a kernel recorded an error status (bounded wait ran out) */
    S1_ENOMEM = -5,
    S1_ELIMIT = -6,   /* s1_linear_static only: the problem is larger than that entry point supports */
    S1_ETIMEOUT = -7  /* a host-side deadline passed (s1_comm_init: a rank never joined) */
};

/* Epilogue fused behind the contraction. */
enum {
    S1_EPI_NONE = 0,   /* y = x W^T                                                                         */
    S1_EPI_GEGLU = 1,  /* w is [2I, K]; y[:, c] = bf16(bf16(gelu_erf(p[:, c])) * p[:, c + I]), c < I          */
    S1_EPI_SWIGLU = 2  /* w = gate_proj [I, K], w_up = up_proj [I, K]; y = bf16(bf16(silu(x Wg^T)) * x Wu^T) */
};

/* Activation applied after the bias (S1_EPI_NONE only). */
enum { S1_ACT_NONE = 0, S1_ACT_RELU = 1, S1_ACT_GELU = 2 };

/*
 * Replaces `device::load` (src/device.rs:43-56, which always opens device 0): opens GPU `device_ordinal`.
 * `cuda_stream` is the cudaStream_t every call of this context enqueues on; NULL is CUDA's default stream.
 * The stream stays the caller's.
 */
int s1_ctx_create(int device_ordinal, void* cuda_stream, s1_ctx** out);
int s1_ctx_destroy(s1_ctx* ctx);
const char* s1_last_error(const s1_ctx* ctx);
/* Joins the stream; returns S1_EKERNEL if any kernel since the last sync recorded an error. */
int s1_sync(s1_ctx* ctx);
/* Number of GPUs visible (replaces the single-device assumption of src/device.rs:48-51). */
int s1_device_count(int* out);
/* Number of kernels this context has launched so far. */
long long s1_launch_count(const s1_ctx* ctx);
/* Tuning knobs: "gemm_bn" = 0 (auto), 512 / 384 (CTA-pair 256x256 / 256x192 tiles), 256 or 128 (single-CTA 128xBN tiles);
 * "gemm_sms" = how many SMs the projections' persistent grids may occupy (0 = all; e.g. 132 leaves 16 SMs to the
 * exchange of the previous slab in a tensor-parallel layer); "comm_ctas" = how many blocks the collective may use
 * (0 = NCCL's default; takes effect at s1_comm_init); "pdl" = 1 (default) launches the projections with
 * programmatic stream serialization, so that a projection's set-up overlaps the tail of the kernel before it, 0 turns
 * that off; "wait_limit_cycles" = SM clock cycles a single wait inside a projection kernel may last before the kernel
 * gives up and s1_sync reports S1_EKERNEL (default 2e9, about a second); "comm_timeout_ms" = how long s1_comm_init
 * waits for the other ranks before it gives up with S1_ETIMEOUT (default 120000; 0 = for ever); "dynamic_tiles" = 1
 * makes the projections' CTAs draw their tiles from a counter at run time instead of working through fixed shares: a CTA
 * that reaches its SM late, because blocks of a collective running beside the projection were in its way, then finds
 * little left to do, where a fixed share would hold the whole launch back (a few microseconds dearer per launch, so
 * off by default; a separate kernel, built for the 256 x 256 pair tiles that large projections use - other shapes keep
 * their fixed shares; the tensor-parallel layers turn it on around their overlapped sums); "exchange_wait_ms" = how long the
 * symmetric-memory exchange kernel waits for its peers (default 10000). */
int s1_set_option(s1_ctx* ctx, const char* name, long long value);

/*
 * Failure-detection self test. Launches a one-block kernel whose only wait can never be satisfied (nothing is in
 * flight and nothing ever arrives on its barrier), so the bounded wait every kernel of this library goes through runs
 * out after "wait_limit_cycles", the kernel records its status and returns by itself; the next `s1_sync` then reports
 * S1_EKERNEL and the context stays usable. Set "wait_limit_cycles" to a few million first, or the call takes about a
 * second. It has no counterpart in the reference, whose failure handling is host-side only (src/batching.rs:252-281).
 */
int s1_selftest_bounded_wait(s1_ctx* ctx);

/*
 * One projection of the reference: a candle `Linear` (weight [N, K] as `vb.get((output, input), "weight")`
 * stores it, src/archs/modernbert.rs:1036-1046, src/archs/qwen35_text.rs:174-176) plus what follows it.
 * `ldw` lets a tensor-parallel rank pass a row range (column-parallel) or a K range (row-parallel) of the
 * full matrix without copying it.
 */
typedef struct s1_linear_desc {
    const void* w;     /* bf16 [N, K], row stride ldw                                              */
    long long ldw;
    const void* w_up;  /* S1_EPI_SWIGLU only: up_proj bf16 [N, K], row stride ldw_up; else NULL    */
    long long ldw_up;
    const void* bias;  /* bf16 [N] or NULL (S1_EPI_NONE only)                                      */
    int N;             /* rows of w; S1_EPI_GEGLU: N = 2 I                                          */
    int K;
    int epilogue;      /* S1_EPI_*                                                                 */
    int act;           /* S1_ACT_*                                                                 */
} s1_linear_desc;

/*
 * y[T, N_out] = epilogue(x[T, K] W^T) (+ residual), N_out = N (S1_EPI_NONE, S1_EPI_SWIGLU) or N / 2 (GEGLU).
 * Rounding follows the reference op by op: the contraction accumulates in f32 and is rounded to bf16 (candle's
 * bf16 matmul), the bias / activation / gate product / residual add each round to bf16 again
 * (src/kernels/modernbert.cu:11-13; src/archs/modernbert.rs:882-886; src/archs/qwen35_text.rs:238-239,938-939).
 * Replaces: modernbert `Attention::forward` Wqkv / Wo (src/archs/modernbert.rs:184-191), `Mlp::forward`
 * (:521-533), qwen35 `Mlp::forward` (src/archs/qwen35_text.rs:232-240), q/k/v/o_proj (:314-339,410),
 * in_proj_* / out_proj (:516,567-568,605-628) and the biased head Linears (src/models/laya.rs:133-155).
 * T is the packed token count (any value >= 1); K and N_out must be multiples of 8.
 * `residual` may be the same buffer as `y` (same leading dimension): the residual stream is then updated in
 * place, `y += x W^T`, which is what the reference's `xs = (xs + ...)` amounts to once the old value is dead.
 */
int s1_linear(s1_ctx* ctx, const s1_linear_desc* lin, const void* x, long long ldx, const void* residual,
              long long ldr, void* y, long long ldy, int T);

/*
 * The projection for callers that cannot allocate device memory. It has no counterpart in the reference: it
 * exists for hosts whose GPU memory is owned by another allocator (sys1's Rust side takes every buffer from
 * candle's pool), and for code running while a stream is captured or inside a latency-critical loop, where
 * cudaMalloc is forbidden or stalls the device. `s1_linear` needs a context, and `s1_ctx_create` allocates the
 * kernels' status block; this entry point needs neither. Its only scratch - that status block - is a 256-byte
 * `__device__` array inside the library (one per GPU that loads it, held until the process exits), and it
 * calls no cudaMalloc / cudaFree or any other allocating routine; tensor maps are encoded on the stack per call.
 *
 * Same arguments and results as `s1_linear` for S1_EPI_NONE (with or without `residual`, in place or not),
 * S1_EPI_GEGLU and S1_EPI_SWIGLU; `bias` and `act` are not offered here. `cuda_stream` is the stream to enqueue
 * on (NULL = default stream). `wait` != 0 makes the call join the stream and return S1_EKERNEL if the kernel
 * recorded an error; with `wait` == 0 the call is asynchronous and a kernel-side error goes unreported.
 * `err` / `err_len`: optional buffer that receives the message of a failing call.
 * Limits: T <= S1_STATIC_MAX_TOKENS, N and K <= S1_STATIC_MAX_FEATURES; beyond them the call returns S1_ELIMIT.
 * The call makes `device_ordinal` current while it runs and puts the caller's current device back before it returns.
 * The first call on a GPU looks up the array's device address and sets kernel attributes: make that first call
 * outside any stream capture. Every call shares the one array (each call clears the status words it needs
 * zeroed), so calls whose kernels may overlap on the GPU - other streams, other threads - race on it: keep the
 * calls of this entry point on one stream at a time.
 */
#define S1_STATIC_MAX_TOKENS 262144
#define S1_STATIC_MAX_FEATURES 32768
int s1_linear_static(int device_ordinal, void* cuda_stream, const s1_linear_desc* lin, const void* x, long long ldx,
                     const void* residual, long long ldr, void* y, long long ldy, int T, int wait, char* err,
                     size_t err_len);

/*
 * Gated delta rule over a token-packed batch; exact drop-in for `chunked_delta_rule(q, k, v, g, beta)`
 * (src/archs/qwen35_text.rs:789-807; CUDA kernel src/kernels/qwen35.cu:53-97), all f32:
 *     S *= exp(g_t);  r = S^T k_t;  delta = (v_t - r) * beta_t;  S += k_t delta^T;  o_t = S^T q_t,   S0 = 0
 * per (sequence, head). q, k: [total_tokens, heads, key_dim] already L2-normalised / scaled as
 * `delta_inputs` leaves them (src/archs/qwen35_text.rs:528-579); v, out: [total_tokens, heads, value_dim];
 * g, beta: [total_tokens, heads]; cu_seqlens: DEVICE int32 [num_seqs + 1], the state restarts at every boundary.
 * (The reference takes [batch, heads, length, dim]; a padded batch is the packed layout with equal lengths after
 * swapping the head and token axes.) key_dim must be 128 (as in the reference's CUDA path, :747), value_dim a
 * multiple of 4.
 */
int s1_delta_rule(s1_ctx* ctx, const float* q, const float* k, const float* v, const float* g, const float* beta,
                  const int32_t* cu_seqlens, int num_seqs, int total_tokens, int heads, int key_dim, int value_dim,
                  float* out);

/*
 * The same recurrence in chunk form on the tensor cores (64-token chunks, bf16 operands, f32 accumulation and f32
 * state): the form of the reference's CPU fallback (src/archs/qwen35_text.rs:809-880), which it evaluates in f32.
 * Results agree with `s1_delta_rule` to bf16 operand precision (relative 2e-2 of the output scale is the bound the
 * tests hold it to), not to 1e-4. key_dim = value_dim = 128 only. `cu_seqlens_host` is a HOST array here (the chunk
 * tables are built on the host; NULL while a batch plan for this batch is in use); `workspace` is device memory, 1024-byte aligned, of at least
 * `s1_delta_rule_chunked_workspace(num_seqs, total_tokens, heads)` bytes, owned by the caller.
 */
size_t s1_delta_rule_chunked_workspace(int num_seqs, int total_tokens, int heads);
int s1_delta_rule_chunked(s1_ctx* ctx, const float* q, const float* k, const float* v, const float* g,
                          const float* beta, const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, int heads,
                          int key_dim, int value_dim, float* out, void* workspace, size_t workspace_bytes);

/*
 * The stages around the recurrence in the Qwen3.5 linear-attention layer, on the packed layout (key dim = value
 * dim = 128; bf16 activations, f32 recurrence inputs):
 *  s1_conv_silu     y = silu(causal depthwise conv(x)) with weight [channels, taps] (the reference's [C, 1, taps]),
 *                   the sum and each product rounded to bf16 tap by tap as in src/kernels/qwen35.cu:3-29
 *                   (CPU form src/archs/qwen35_text.rs:632-650). `positions` (DEVICE int32 [T], index of each token
 *                   inside its own sequence, from s1_pack_batch) gives the zero left padding per sequence.
 *                   y must not overlap x (S1_EINVAL): a token reads the rows before it.
 *  s1_delta_inputs  `delta_inputs` (src/archs/qwen35_text.rs:528-579): split mixed = [q | k | v], repeat the key
 *                   heads over the value heads, q = l2norm(q) / sqrt(128), k = l2norm(k) (1e-6 inside the root),
 *                   beta = sigmoid(b), g = softplus(a + dt_bias) * neg_exp_a; outputs f32 [T, Hv, 128] / [T, Hv].
 *  s1_delta_finish  `finish_delta` up to out_proj (:597-626): o / sqrt(mean(o^2) + eps) * norm_weight * silu(z) -> bf16.
 *  s1_gated_delta_rule  the three in a row around s1_delta_rule_chunked, from the conv output to the out_proj
 *                   input; `workspace` (device, 1024-byte aligned) of s1_gated_delta_rule_workspace(...) bytes.
 *                   Its recurrence is the chunk form (bf16 operands, f32 state): within 2e-2 of the output scale of the
 *                   exact f32 recurrence, not within the reference's 1e-4; s1_delta_inputs -> s1_delta_rule ->
 *                   s1_delta_finish is the same path at the reference's own precision.
 *  s1_gated_delta_rule_conv  s1_conv_silu (4 taps) and s1_gated_delta_rule as one call: `mixed_before_conv` is the
 *                   projection the conv would read, `conv_weight` [2 * key_heads * 128 + value_heads * 128, 4] bf16
 *                   (16-byte aligned), `positions` as for s1_conv_silu. The recurrence's first kernel applies conv + SiLU to
 *                   the rows it stages (with three rows of history per 64-token chunk), so the conv's pass over the
 *                   [T, channels] tensor and back is never made; the result is bit-identical to the two calls.
 */
int s1_conv_silu(s1_ctx* ctx, const void* x, long long ldx, const void* weight, const int32_t* positions, int total_tokens,
                 int channels, int taps, void* y, long long ldy);
int s1_delta_inputs(s1_ctx* ctx, const void* mixed, long long ldm, const void* b_proj, const void* a_proj, long long ldba,
                    const float* dt_bias, const float* neg_exp_a, int total_tokens, int key_heads, int value_heads, float* q,
                    float* k, float* v, float* g, float* beta);
int s1_delta_finish(s1_ctx* ctx, const float* o, const void* z, long long ldz, const void* norm_weight, float eps,
                    int total_tokens, int value_heads, void* y, long long ldy);
size_t s1_gated_delta_rule_workspace(int num_seqs, int total_tokens, int value_heads);
int s1_gated_delta_rule(s1_ctx* ctx, const void* mixed, long long ldm, const void* b_proj, const void* a_proj, long long ldba,
                        const float* dt_bias, const float* neg_exp_a, const void* z, long long ldz, const void* norm_weight,
                        float eps, const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, int key_heads,
                        int value_heads, void* y, long long ldy, void* workspace, size_t workspace_bytes);
int s1_gated_delta_rule_conv(s1_ctx* ctx, const void* mixed_before_conv, long long ldm, const void* conv_weight,
                             const int32_t* positions, const void* b_proj, const void* a_proj, long long ldba, const float* dt_bias,
                             const float* neg_exp_a, const void* z, long long ldz, const void* norm_weight, float eps,
                             const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, int key_heads, int value_heads, void* y,
                             long long ldy, void* workspace, size_t workspace_bytes);

/*
 * Batch plan: the tables the attention and delta-rule kernels walk - the 128-query blocks of every sequence in the order
 * each attention kernel starts them, and the 64-token chunks of the delta rule - built once per packed batch instead of
 * once per kernel call. Every layer of a stack sees the same batch, so the per-call form costs one small host-to-device
 * copy per layer and keeps those calls out of CUDA graphs; the reference likewise derives its `cu_seqlens` once per batch
 * (src/archs/modernbert.rs:431-443).
 *   s1_batch_plan_bytes : size of the device buffer a plan needs
 *   s1_batch_plan       : builds the tables from the HOST offsets and copies them into `plan` (device memory, 256-byte
 *                         aligned, owned by the caller) on the context's stream
 *   s1_use_batch_plan   : makes a plan built on this context the one in use (NULL: none). While a plan is in use,
 *                         s1_attention, s1_attention_gqa, s1_delta_rule_chunked and s1_gated_delta_rule may be called
 *                         with `cu_seqlens_host` = NULL for the same (num_seqs, total_tokens): they then read their
 *                         tables from the plan and copy nothing (the attentions need no workspace then).
 *   s1_batch_plan_release : the context forgets the plan built in this buffer (if it is the one in use, none is in use
 *                         afterwards); call it before the buffer is freed or reused for something else. Building a new
 *                         plan in the same buffer replaces the old one without a release. A context keeps up to 4096
 *                         plans alive; s1_batch_plan fails with S1_EINVAL beyond that.
 * The caller keeps the buffer alive and unchanged while the plan is in use. A call that does pass `cu_seqlens_host`
 * ignores the plan and behaves as before (and refuses to run under stream capture, where its copy from host memory
 * would be recorded with a pointer that does not outlive the call).
 */
size_t s1_batch_plan_bytes(int num_seqs, int total_tokens);
int s1_batch_plan(s1_ctx* ctx, const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, void* plan, size_t plan_bytes);
int s1_use_batch_plan(s1_ctx* ctx, const void* plan);
int s1_batch_plan_release(s1_ctx* ctx, const void* plan);

/*
 * Bidirectional softmax attention over a packed batch in flash form (scores stay on chip), head_dim = 64:
 *     out_i = sum_j softmax_j(scale * q_i . k_j) v_j   over the keys j of the same sequence with |i - j| <= window
 * (`window` < 0: all keys of the sequence). This is `scaled_dot_product_attention` of the reference
 * (src/archs/modernbert.rs:313-351) with its local mask (:1058-1076, window = local_attention / 2); the packed
 * layout has no padded keys, so the global mask (:1048-1056) has nothing to mask. q, k, v: bf16 [T, heads * 64]
 * views with row strides ldq / ldk / ldv (they may be the three column blocks of the Wqkv output, after RoPE);
 * out: bf16 [T, heads * 64] = the merged-heads layout Wo consumes (`merge_heads`, :249-260).
 * `cu_seqlens_host`: HOST int32 [num_seqs + 1]; `workspace`: device memory of s1_attention_workspace(...) bytes
 * (both may be NULL while a batch plan for this batch is in use). `scale` must be positive.
 * Softmax in f32, probabilities rounded to bf16 before they multiply V (as the reference does, :349-350).
 */
size_t s1_attention_workspace(int num_seqs, int total_tokens);
int s1_attention(s1_ctx* ctx, const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                 const int32_t* cu_seqlens_host, int num_seqs, int total_tokens, int heads, int head_dim, int window,
                 float scale, void* out, long long ldo, void* workspace, size_t workspace_bytes);

/*
 * Causal grouped-query softmax attention over a packed batch in flash form, head_dim = 256: the attention core of
 * the reference's `FullAttention::forward` (src/archs/qwen35_text.rs:312-411),
 *     a_i = sum_{j <= i} softmax_j(scale * q_i . k_j) v_j     over the keys j of the same sequence,
 * query head h reading KV head h / (heads / kv_heads) (`repeat_kv`, :363-369), with the layer's output gate fused
 * into the write-out when `gate` is not NULL: out = bf16(a) * bf16(sigmoid(gate)) (:325-329, :408).
 * q: bf16, head h of token t at q + t * ldq + h * q_head_stride (so the query halves of the interleaved q_proj
 * output, [T, heads, 2, 256], are read in place with q_head_stride = 512, and gate = q + 256 likewise);
 * k, v: bf16 [T, kv_heads * 256] views with their own strides; out: bf16 [T, heads * 256] (what o_proj consumes).
 * `cu_seqlens_host`: HOST int32 [num_seqs + 1]; `workspace`: device memory of s1_attention_gqa_workspace(...) bytes
 * (both may be NULL while a batch plan for this batch is in use). `scale` must be positive.
 */
size_t s1_attention_gqa_workspace(int num_seqs, int total_tokens);
int s1_attention_gqa(s1_ctx* ctx, const void* q, long long ldq, long long q_head_stride, const void* k, long long ldk,
                     long long k_head_stride, const void* v, long long ldv, long long v_head_stride, const void* gate,
                     long long ldg, long long gate_head_stride, const int32_t* cu_seqlens_host, int num_seqs,
                     int total_tokens, int heads, int kv_heads, int head_dim, float scale, void* out, long long ldo,
                     void* workspace, size_t workspace_bytes);

/*
 * Row-wise normalisation of a bf16 matrix, statistics in f32, one rounding at the end:
 *     kind 0  y = (x - mean(x)) / sqrt(var(x) + eps) * weight (+ bias)   LayerNorm: without bias the reference's `Norm`
 *                                                                    (src/archs/modernbert.rs:1006-1034), with `bias`
 *                                                                    (bf16 [width], else NULL) the `layer_norm` of the
 *                                                                    decision heads (src/models/laya.rs:85-86,258)
 *     kind 1  y = x / sqrt(mean(x^2) + eps) * (1 + weight)           the reference's `RmsNorm`
 *                                                                    (src/archs/qwen35_text.rs:178-203)
 *     kind 2  y = x                                                  no normalisation (weight, bias, eps unused): with
 *                                                                    `gather` the plain embedding lookup of the decoder
 *                                                                    (`Decoder::embed`, src/archs/qwen35_text.rs:978-980)
 * x: [rows, width] with row stride ldx; weight: bf16 [width]; y: [rows, width] with row stride ldy (may be x).
 * With `gather` (DEVICE int32 [rows]) row r is read from x[gather[r]]: the embedding lookup fused with the
 * embedding norm (src/archs/modernbert.rs:1084-1092); `gather_rows` is the row count of x, and an index outside
 * it is reported by s1_sync as S1_EKERNEL (that row is left unwritten); the same index is the marker-row selection
 * ahead of the scorer (`index_select` + `scorer_norm`, src/models/laya.rs:476-513). Rows of any width that is a multiple of 8:
 * hidden states (rows = tokens) and per-head q / k norms (rows = tokens x heads, width = head_dim) alike.
 */
int s1_norm(s1_ctx* ctx, const void* x, long long ldx, const int32_t* gather, int gather_rows, const void* weight,
            const void* bias, float eps, int kind, void* y, long long ldy, long long rows, int width);

/*
 * y[r, :] = bf16(x[r, :] + table[index[r], :]): a row of a small table added to every row of x, chosen by a DEVICE
 * int32 index [rows]. The type-embedding add of the decision model (`hidden.broadcast_add(type_ids.apply(&type_embedding))`,
 * src/models/laya.rs:431) on the packed layout: index[r] is the question kind of the sequence token r belongs to.
 * x, y: bf16 [rows, width] (y may be x); table: bf16 [table_rows, width]. An index outside the table is reported by
 * s1_sync as S1_EKERNEL (that row is left unwritten).
 */
int s1_add_rows(s1_ctx* ctx, const void* x, long long ldx, const void* table, long long ldt, const int32_t* index,
                int table_rows, void* y, long long ldy, long long rows, int width);

/*
 * Rotate-half rotary embedding, in place, on `heads` consecutive heads of every token row:
 *     lo' = lo * cos - hi * sin,  hi' = lo * sin + hi * cos     for the column pairs (j, j + rotary_dim / 2)
 * of the first `rotary_dim` columns of each head; the rest of the head is left as it is. x: bf16 [T, ldx], head h
 * of token t starts at x + t * ldx + h * head_stride. cos_table / sin_table: DEVICE f32
 * [max_positions, rotary_dim / 2]; positions: DEVICE int32 [T], a position outside the table is reported by
 * s1_sync as S1_EKERNEL (that token is left unrotated). Replaces `rope_qkv` (src/kernels/modernbert.cu:31-62,
 * called from `RotaryEmbedding::apply_qkv`): on the packed Wqkv output [T, 3 * H * D] call it with heads = 2 * H
 * (q and k lie side by side); v stays where it is and s1_attention reads the three column blocks in place.
 * Also `Attention::rotary` of src/archs/qwen35_text.rs:296-310 (rotary_dim < head_dim) with the products and the sum
 * formed in f32 and rounded once, which is the arithmetic of the ModernBERT kernel; s1_head_norm_rope offers the
 * per-operation bf16 rounding candle applies on that path.
 */
int s1_rope(s1_ctx* ctx, void* x, long long ldx, const float* cos_table, const float* sin_table, const int32_t* positions,
            int max_positions, int total_tokens, int heads, long long head_stride, int rotary_dim);

/*
 * Per-head RMSNorm followed by the partial rotary embedding, in place, one pass: `q_norm` / `k_norm` and
 * `Attention::rotary` of the reference's `FullAttention::forward` (src/archs/qwen35_text.rs:296-339):
 *     y = bf16(x / sqrt(mean(x^2) + eps) * (1 + norm_weight))   over the head_dim columns of each (token, head)
 *     then the rotate-half rotation of s1_rope on the first rotary_dim columns of y.
 * x: bf16, head h of token t at x + t * ldx + h * head_stride (the query halves of the interleaved q_proj output with
 * head_stride = 2 * head_dim, or the k_proj output with head_stride = head_dim). head_dim 64, 128 or 256; rotary_dim
 * 16, 32, 64, 128 or 256 (<= head_dim). Tables and positions as for s1_rope.
 * bf16_ops != 0: the rotation rounds as candle's bf16 tensor ops do - each product and the sum is a bf16 value
 * (x * cos, rotate_half(x) * sin, their sum: three roundings, :302); bf16_ops = 0: products and sum in f32, one
 * rounding, bit-identical to s1_norm followed by s1_rope.
 */
int s1_head_norm_rope(s1_ctx* ctx, void* x, long long ldx, long long head_stride, int heads, int head_dim,
                      const void* norm_weight, float eps, const float* cos_table, const float* sin_table,
                      const int32_t* positions, int max_positions, int rotary_dim, int total_tokens, int bf16_ops);

/*
 * Tensor parallelism: the sum over ranks that follows a row-parallel projection (each rank holds a K range of the
 * weight and produces a partial [T, N]). The reference has no multi-GPU path (`device::load` opens GPU 0 only,
 * src/device.rs:43-56); these entry points exist for the sharded projections of the large hybrid model.
 * NCCL over NVLink underneath, looked up at run time (libnccl.so.2); single-GPU callers never need it.
 *   s1_comm_unique_id : rank 0 makes the 128-byte id every rank passes to s1_comm_init (carry it over any channel)
 *   s1_comm_init      : collective over all `size` ranks, one context (= one GPU) per rank
 *   s1_allreduce_bf16 : in-place sum of `count` bf16 values over the ranks. Runs on a communication stream of the
 *                       context's own, after everything queued on the context's stream so far; returns at once.
 *                       Called slab by slab it overlaps the exchange of one slab with the projection of the next.
 *   s1_allreduce_wait : orders the context's stream after every all-reduce issued so far (no host blocking)
 *   s1_allreduce_ticket / s1_allreduce_wait_ticket : the sequence number of the all-reduce issued last (1, 2, ...), and
 *                       the wait for one of them only: the context's stream is ordered after that all-reduce and not
 *                       after the ones issued later, so that two micro-batches can alternate - one computes while the
 *                       other's sum travels
 *   s1_comm_destroy   : also done by s1_ctx_destroy
 * Every rank must issue the same sequence of all-reduces with the same counts.
 */
#define S1_COMM_ID_BYTES 128
int s1_comm_unique_id(void* id_out, char* err, size_t err_len);
int s1_comm_init(s1_ctx* ctx, const void* id, int rank, int size);
int s1_comm_destroy(s1_ctx* ctx);
int s1_allreduce_bf16(s1_ctx* ctx, void* buf, size_t count);
int s1_allreduce_wait(s1_ctx* ctx);
long long s1_allreduce_ticket(const s1_ctx* ctx);
int s1_allreduce_wait_ticket(s1_ctx* ctx, long long ticket);

/*
 * Symmetric-memory exchange: `s1_exchange_register` tells the context that [local_base, local_base + bytes) is symmetric
 * memory - the same buffer allocated on every rank, with `multicast_base` the address of its NVLink multicast mapping
 * (for instance from torch.distributed._symmetric_memory, or cuMulticast* directly) - and hands it one small flag array
 * per rank (`flag_arrays_host`: HOST array of `size` DEVICE pointers, entry r = rank r's array as mapped on this GPU, each
 * of at least S1_EXCHANGE_FLAG_BYTES, zeroed by its owner before the first sum). From then on s1_allreduce_bf16 on a
 * buffer inside that range runs this library's own kernel instead of the NCCL call: every rank reduces its slice inside the
 * NVSwitch (`multimem.ld_reduce`, f32 accumulation, one rounding) and writes the sums into every rank's copy
 * (`multimem.st`); per GPU (1 + 1 / ranks) buffers of NVLink traffic in each direction, whatever the number of ranks;
 * a few blocks of 1024 threads ("comm_ctas": how many, by default 16 for two ranks and 8 for four or more, at most 64), so that the projections running beside the
 * sum lose few SMs to it; bit-identical results on all ranks. Tickets
 * and waits work as for the NCCL path; a context that only sums symmetric buffers needs no s1_comm_init. The ranks meet
 * through the flag arrays with bounded polls: a rank that never shows up makes the others give up after
 * "exchange_wait_ms" (s1_set_option, default 10000) and s1_sync report S1_EKERNEL; the context stays usable. The
 * ranks' epoch counters no longer agree after that: before summing again every rank zeroes its flag array and registers
 * anew (which restarts the epochs).
 * `size` = 0 forgets the registration (the other arguments are ignored). The caller keeps the memory mapped until then.
 */
#define S1_EXCHANGE_FLAG_BYTES 4096
int s1_exchange_register(s1_ctx* ctx, int rank, int size, void* local_base, void* multicast_base, size_t bytes,
                         void* const* flag_arrays_host, size_t flag_bytes);

/*
 * s1_linear followed by s1_rope on the first `rotated_heads` heads (64 columns each) of the output, the rotation done
 * in the projection's epilogue while the tile is still on chip: the reference's Wqkv projection and its `rope_qkv`
 * kernel (src/archs/modernbert.rs:184-205, src/kernels/modernbert.cu:31-62) as one launch. Plain projections only
 * (no bias, activation, gating or residual); head_dim = rotary_dim = 64. The result is bit-identical to the two calls
 * made one after the other, which is also what happens for shapes the fused tile does not cover (fewer than a wave of
 * 256 x 256 tiles, or a rotated width that is not a multiple of 128 columns).
 */
int s1_linear_rope(s1_ctx* ctx, const s1_linear_desc* lin, const void* x, long long ldx, void* y, long long ldy, int T,
                   const float* cos_table, const float* sin_table, const int32_t* positions, int max_positions,
                   int rotated_heads);

/*
 * Packs the next sequences of a queue into one token-packed batch (host arrays, no GPU work).
 * Takes sequences in order while the running token count stays within `token_budget`; a sequence longer than
 * the budget forms a batch of its own. Writes cu_seqlens[0..num_taken] (cu_seqlens[0] = 0, last = total) and,
 * if `positions_host` is not NULL, positions[t] = index of token t within its own sequence.
 * `padded_tokens` = total rounded up to `pad_multiple` (rows total..padded are padding the caller zero-fills).
 * Stands where the reference pads to [batch, max_len] (src/models/laya.rs:396-431) after its request batcher
 * (src/batching.rs:83-102); cu_seqlens has the layout of src/archs/modernbert.rs:431-443.
 */
int s1_pack_batch(const int32_t* lengths_host, int num_sequences, int token_budget, int pad_multiple,
                  int32_t* cu_seqlens_host, int32_t* positions_host, int* num_taken, int* total_tokens,
                  int* padded_tokens);

#ifdef __cplusplus
}
#endif
#endif /* SYS1_B200_H_ */

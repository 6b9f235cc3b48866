/* lm_b200.h - C ABI of the decoder-only language-model path (liblm_b200.so, sm_100a).
 *
 * Same conventions as dia_b200.h: plain C types, device pointers, an explicit CUDA stream passed as void*, 0 on
 * success or a negative code, nothing throws, a forward call neither allocates nor synchronises.  There is no CPU
 * fallback: every compute entry point launches kernels.
 *
 * A model is a stack of layers  x += norm_b(mixer(tapmix(norm_a(x))));  x += norm_b'(ff(tapmix'(norm_a'(x))))  described
 * by lm_b200_layer records: the mechanisms are selected and parameterised per layer, so another design can combine them
 * differently.  Matrices are bf16 [out][in]; vectors and scalars fp32.  The residual stream, norms, the router,
 * attention scores and the K/V pages are fp32; the operands of the matrix products are fp32 or bf16 (lm_b200_precision).
 *
 * A step is a flat batch of M rows (the new tokens of the scheduled sequences, the rows of one sequence adjacent and in
 * order) described by one int32 device buffer:
 *     token[M] | slot[M] | pos[M] | start[M] | seq_slot[S] | seq_row0[S] | seq_count[S] | want[W]
 * slot: the sequence's state slot; pos: position in its sequence; start: position of the sequence's first row in this
 * step; seq_*: per scheduled sequence its slot, first row and row count; want: rows whose logits are returned.
 */
#ifndef LM_B200_H
#define LM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LM_B200_ABI_VERSION 1

enum lm_b200_status { LM_B200_OK = 0, LM_B200_EINVAL = -1, LM_B200_ECUDA = -2, LM_B200_ENOMEM = -3, LM_B200_EUNSUPPORTED = -5 };

enum lm_b200_mixer_kind { LM_B200_MIXER_SINK_ATTENTION = 1 };
enum lm_b200_ff_kind { LM_B200_FF_NONE = 0, LM_B200_FF_ROUTED_EXPERTS = 1 };
/* FP32: every product is fp32 FMA arithmetic on the stored weights.  BF16: the products of a long step (a prompt portion)
 * run on the tensor cores with bf16 operands and fp32 accumulation; everything else stays fp32. */
enum lm_b200_precision { LM_B200_PRECISION_FP32 = 0, LM_B200_PRECISION_BF16 = 1 };

/* DynamicTanh norm: y = tanh(alpha x) w + b */
typedef struct lm_b200_norm {
    const float *w, *b;
    float alpha;
    int32_t reserved;
} lm_b200_norm;

typedef struct lm_b200_layer {
    int32_t mixer;                 /* lm_b200_mixer_kind */
    int32_t heads, kv_heads, dim;  /* query heads, key/value heads, per-head size (values are the projected keys) */
    int32_t window, keep_first;    /* key j <= i is seen when i - j < window or j < keep_first; window <= 0: all */
    float scale, softcap;          /* score multiplier; tanh cap (<= 0: none) */
    int32_t ff;                    /* lm_b200_ff_kind */
    int32_t experts, top, expert_ff, shared_ff; /* shared_ff 0: no shared expert */
    lm_b200_norm norm_mix_in, norm_mix_out, norm_ff_in, norm_ff_out;
    const float *tap_mix, *tap_ff; /* [width][taps] causal per-channel taps in front of each sublayer; NULL: none */
    const void *w_qk;              /* [(heads + kv_heads) * dim][width]: query rows, then key rows */
    const float *q_norm, *k_norm;  /* whole-projection RMS norm weights */
    const float *temp, *slopes, *sink; /* per query head: score temperature, distance-bias slope, sink logit (NULL: none) */
    const void *w_o;               /* [width][heads * dim] */
    const void *w_router;          /* [experts][width] */
    const void *w_gate_up;         /* [experts][2 * expert_ff][width]: gate rows, then up rows */
    const void *w_down;            /* [experts][width][expert_ff] */
    const void *ws_gate_up, *ws_down; /* the shared expert, same form with shared_ff */
    float *k_pages, *v_pages;      /* [pages][kv_heads][page_size][dim] */
    float *tail_mix, *tail_ff;     /* [slots][taps - 1][width]: last normed inputs of each sublayer per sequence */
} lm_b200_layer;

typedef struct lm_b200_model {
    int32_t n_layer, width, vocab, taps;
    int32_t page_size, max_pages, n_slots, max_rows; /* max_pages: per sequence; max_rows: rows of one forward call */
    float eps;                     /* inside the root of every RMS norm */
    int32_t precision;             /* lm_b200_precision */
    const void *embed, *head;      /* [vocab][width] */
    lm_b200_norm final_norm;
    const int32_t *page_table;     /* device, [n_slots][max_pages] */
    int32_t step_graphs;           /* != 0: steps of a few rows (decoding) replay a CUDA graph captured at their first use */
    int32_t reserved;
} lm_b200_model;

typedef struct lm_b200_engine lm_b200_engine;

int lm_b200_abi_version(void);
const char *lm_b200_last_cuda_error(void);
int64_t lm_b200_launch_count(void);

/* Copies the descriptors and allocates the step workspace for max_rows rows.  The weights, pages, tails and the page
 * table stay the caller's memory. */
int lm_b200_engine_create(const lm_b200_model *model, const lm_b200_layer *layers, int device, lm_b200_engine **out);
int lm_b200_engine_destroy(lm_b200_engine *e);
size_t lm_b200_engine_workspace_bytes(const lm_b200_engine *e);

/* One step: embeds the rows, runs every layer (appending to the pages and tails of the rows' sequences), and writes the
 * logits of the wanted rows, float32 [n_want][vocab].  layers_out (optional): the residual stream after every layer,
 * float32 [n_layer][M][width]. */
int lm_b200_forward(lm_b200_engine *e, const int32_t *step, int M, int n_seq, int n_want, float *logits_out,
                    float *layers_out, void *stream);

/* ---- the mechanisms one at a time (operator boundaries; `step` has the layout above with n_want = 0) ---- */
/* out = tapmix(norm_in(x)) of sublayer `sub` (0 mixer, 1 feed-forward) of `layer`, and the tail update */
int lm_b200_op_norm_tapmix(lm_b200_engine *e, int layer, int sub, const float *x, const int32_t *step, int M, int n_seq,
                           float *out, void *stream);
/* y = mixer(h): projections, norms, page append, attention, output projection */
int lm_b200_op_mixer(lm_b200_engine *e, int layer, const float *h, const int32_t *step, int M, int n_seq, float *y,
                     void *stream);
/* attention alone on projected rows qk [M][(heads + kv_heads) * dim] (query part, then key part): the whole-projection
 * norms (q in place), the page append and the attention; out [M][heads * dim] */
int lm_b200_op_attention(lm_b200_engine *e, int layer, float *qk, const int32_t *step, int M, int n_seq, float *out,
                         void *stream);
/* y = ff(h): router, expert groups, shared expert; the sum over a row's experts */
int lm_b200_op_ff(lm_b200_engine *e, int layer, const float *h, int M, float *y, void *stream);
/* Y[M][N] = A[M][K] . W[N][K]^T */
int lm_b200_op_linear(const float *A, const void *W_bf16, float *Y, int M, int N, int K, void *stream);
/* the same on the tensor cores: A is rounded to bf16 into a_bf16 [M][K] first.  K a multiple of 8, N of 4, else
 * LM_B200_EUNSUPPORTED */
int lm_b200_op_linear_tc(const float *A, const void *W_bf16, float *Y, void *a_bf16, int M, int N, int K, void *stream);
/* greedy sampling: out[r] = index of the largest of logits[r][0 .. V) (ties: the lowest index) */
int lm_b200_argmax_rows(const float *logits, int M, int V, int32_t *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif

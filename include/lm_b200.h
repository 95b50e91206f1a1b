/* lm_b200.h - C ABI of the decoder-only language-model path (liblm_b200.so, sm_100a).
 *
 * Same conventions as dia_b200.h: plain C types, device pointers, an explicit CUDA stream passed as void*, 0 on
 * success or a negative code, nothing throws, a forward call neither allocates nor synchronises.  There is no CPU
 * fallback: every compute entry point launches kernels.
 *
 * A model is a stack of layer records.  A record has one of three forms:
 *   sequential  x += norm_b(mixer(tapmix(norm_a(x))));  x += norm_b'(ff(tapmix'(norm_a'(x))))
 *   parallel    h = norm_a(x);  x += mixer(h) + ff(h)
 *   streams     s residual streams x_1 .. x_s (all equal to the embedding output at first, summed at the end); per sublayer
 *               u = sum_s in[s] x_s;  y = sublayer(norm(u));  x_j <- sum_s mix[s][j] x_s + out[j] y   (hyper-connections;
 *               s = 1 with unit weights is the plain pre-norm residual)
 *               with `parallel`, both sublayers read the streams before either writes: x += mixer(norm1(x)) + ff(norm2(x))
 * and the mechanisms (norm kind, mixer kind, feed-forward kind) are selected and parameterised per record, so a design
 * combines them as it needs.  A layer that a design runs several times with the same weights is several records that
 * share weight pointers and differ in their state pointers.  Matrices are bf16 [out][in]; vectors and scalars fp32.
 * The residual stream, norms, the router, attention scores, the K/V pages, recurrent states and everything that enters
 * a recurrence are fp32; the operands of the matrix products are fp32 or bf16 (lm_b200_precision).
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

#define LM_B200_ABI_VERSION 4

enum lm_b200_status { LM_B200_OK = 0, LM_B200_EINVAL = -1, LM_B200_ECUDA = -2, LM_B200_ENOMEM = -3, LM_B200_EUNSUPPORTED = -5 };

enum lm_b200_mixer_kind {
    LM_B200_MIXER_SINK_ATTENTION = 1,   /* values = projected keys, whole-projection norms, window, distance bias, sink */
    LM_B200_MIXER_TALK_ATTENTION = 2,   /* biased q/k/v, per-head norms, rotary positions, scores mixed across heads, sink, gate */
    LM_B200_MIXER_HGRN2 = 3,            /* gated linear recurrence: the forget gate also sets the write strength */
    LM_B200_MIXER_CHANNEL_DELTA = 4,    /* gated delta rule with a decay per head and key channel, short convolutions */
    LM_B200_MIXER_LATENT_ATTENTION = 5, /* queries through a normed latent, keys / values up-projected from one cached normed latent, sink, elementwise gate */
    LM_B200_MIXER_MLSTM = 6,            /* matrix memory with exponential input gate, running maximum and normaliser */
    LM_B200_MIXER_GATED_DELTA = 7,      /* gated delta rule with ONE decay per head and token, short convolutions, silu output gate */
    LM_B200_MIXER_RETENTION = 8         /* linear attention with a fixed decay per head, rotary q / k, no softmax, no denominator */
};
enum lm_b200_ff_kind { LM_B200_FF_NONE = 0, LM_B200_FF_ROUTED_EXPERTS = 1, LM_B200_FF_DENSE = 2 };
enum lm_b200_norm_kind { LM_B200_NORM_DYT = 0, LM_B200_NORM_LAYER = 1, LM_B200_NORM_RMS = 2 };
enum lm_b200_layer_form { LM_B200_FORM_SEQUENTIAL = 0, LM_B200_FORM_PARALLEL = 1, LM_B200_FORM_STREAMS = 2 };
/* XIELU: up, activation, down.  SILU_GLU / CLAMPED_GLU: gated units [gate | up] -> down with silu(g) u, or with
 * g' = min(g, limit), u' = clamp(u, -limit, limit): g' sigmoid(1.702 g') (u' + 1) */
enum lm_b200_act_kind { LM_B200_ACT_SILU_GLU = 0, LM_B200_ACT_XIELU = 1, LM_B200_ACT_CLAMPED_GLU = 2,
                        LM_B200_ACT_RELU2 = 3 /* dense, not gated: up, max(z, 0)^2, down */ };
/* SIGMOID_INPUT: score sigmoid(z) multiplies the chosen expert's input.  SOFTMAX_TOP: the softmax over the chosen logits
 * alone weighs the experts' outputs */
/* SOFTMAX_GROUPED: scores = softmax over ALL router outputs; the choice is made on score + correction, only inside the
 * `group_keep` of `group_count` groups of neighbouring outputs whose largest choice score is largest; the chosen scores
 * (without the correction), divided by their sum and times route_scale, weigh the experts' outputs.  The last
 * `identity_experts` router outputs have no weights: their output is their input. */
enum lm_b200_router_kind { LM_B200_ROUTER_SIGMOID_INPUT = 0, LM_B200_ROUTER_SOFTMAX_TOP = 1, LM_B200_ROUTER_SOFTMAX_GROUPED = 2 };
/* what the columns `gate` of a mixer's stacked projections do to its output */
enum lm_b200_gate_kind { LM_B200_GATE_SIGMOID = 0, LM_B200_GATE_NONE = 1, LM_B200_GATE_SILU = 2 };
/* which channels of a head form a rotary pair: (2i, 2i + 1), or (i, i + rot_dims / 2) */
enum lm_b200_rot_layout { LM_B200_ROT_INTERLEAVED = 0, LM_B200_ROT_HALF = 1 };
/* FP32: every product is fp32 FMA arithmetic on the stored weights.  BF16: the products of a long step (a prompt portion)
 * run on the tensor cores with bf16 operands and fp32 accumulation; everything else stays fp32. */
enum lm_b200_precision { LM_B200_PRECISION_FP32 = 0, LM_B200_PRECISION_BF16 = 1 };

/* DYT: y = tanh(alpha x) w + b.  LAYER: y = (x - mean) / sqrt(var + eps) * w + b with the model's eps.
 * RMS: y = x / sqrt(mean(x^2) + eps) * w (stream records, the final norm, the embedding norm). */
typedef struct lm_b200_norm {
    const float *w, *b;
    float alpha;
    int32_t kind;                  /* lm_b200_norm_kind */
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
    float *k_pages, *v_pages;      /* [pages][kv_heads][page_size][dim]; the value pages of a talk attention have [vdim] rows */
    float *tail_mix, *tail_ff;     /* [slots][taps - 1][width]: last normed inputs of each sublayer per sequence */

    /* ---- the parallel form and its mechanisms (all zero / NULL in a sequential record) ---- */
    int32_t form;                  /* lm_b200_layer_form */
    int32_t vdim;                  /* value size per head (the sink attention above has vdim = dim and ignores this) */
    int32_t rot_dims;              /* leading channels of every q / k head that turn with the position (pairs 2i, 2i+1); 0: none */
    int32_t conv_taps;             /* taps of the short causal convolutions of q, k, v (channel delta) */
    int32_t rank_a, rank_g;        /* inner sizes of the two-step decay and gate projections (channel delta) */
    int32_t dense_ff, act;         /* hidden size of the dense feed-forward; lm_b200_act_kind */
    float act_p, act_q;            /* xIELU: z > 0: act_p z^2 + z / 2;  z <= 0: act_q (e^z - 1 - z) + z / 2 */
    float unit_eps;                /* inside the root of the unit-vector norm of q and k (channel delta) */
    int32_t n_in, k_out;           /* rows of w_in (padded to a multiple of 4); columns of w_out */
    /* every projection that reads h, stacked [n_in][width], in this order and then the feed-forward's up rows:
     *   TALK_ATTENTION  q (heads*dim) | k (kv_heads*dim) | v (kv_heads*vdim) | gate (heads)
     *   HGRN2           q (heads*dim) | f (heads*dim) | v (heads*vdim)
     *   CHANNEL_DELTA   q (kv_heads*dim) | k (kv_heads*dim) | v (heads*vdim) | beta (heads) | a1 (rank_a) | g1 (rank_g) */
    const void *w_in;
    const float *in_bias;          /* [n_in] added to the stacked projections where a mechanism has biases; NULL: none */
    const void *w_out;             /* [width][k_out]: the mixer's output projection beside the feed-forward's down projection */
    const void *w_pre;             /* [width][2 width]: x <- w_pre [x; embedding output] before this record; NULL: none */
    const float *rot_freq;         /* [rot_dims / 2] angle per position of every rotary pair */
    const float *talk;             /* [heads][heads] score_h <- sum_g talk[h][g] score_g before the softmax; NULL: none */
    const float *head_norm;        /* [vdim] weight of the per-head RMS norm of a recurrent mixer's read-out */
    const float *lower;            /* [heads*dim] lower bound of the forget gate (HGRN2) */
    const float *conv_w;           /* [2 kv_heads*dim + heads*vdim][conv_taps]: q, k, v channels; the last tap is the current token's */
    const float *a_log, *dt_bias;  /* [heads], [heads*dim]: decay = exp(-exp(a_log_h) softplus(a2 a1 h + dt_bias)) */
    const void *w_a2, *w_g2;       /* bf16 [heads*dim][rank_a], [heads*vdim][rank_g]: second steps of the decay and gate projections (fp32 arithmetic) */
    float *rec_state;              /* [slots][heads][vdim][dim] recurrent state per sequence (column of a value channel contiguous) */
    float *conv_tail;              /* [slots][conv_taps - 1][2 kv_heads*dim + heads*vdim] last projected inputs per sequence */

    /* ---- the stream form and its mechanisms (all zero / NULL in the other forms) ----
     * norm_mix_in / norm_ff_in: layer norms (weight; bias NULL) of the two sublayers.  w_in stacks every projection that
     * reads the mixer's input, [n_in][width] (in_bias as above):
     *   LATENT_ATTENTION  query latent (q_rank) | key/value latent (kv_rank) | gate (heads*vdim)
     *   MLSTM             q (heads*dim) | k (heads*dim) | v (heads*vdim) | input gate (heads) | forget gate (heads) | gate (heads*vdim)
     * w_o [width][heads*vdim] is the output projection.  Feed-forward: FF_DENSE is one gated unit (ws_gate_up / ws_down with
     * dense_ff hidden units and act_limit); FF_ROUTED_EXPERTS as above with router, router_bias, act and the two limits. */
    int32_t streams;               /* residual streams s, 1 .. 8 */
    const float *hc_in[2], *hc_out[2], *hc_mix[2]; /* per sublayer (0 mixer, 1 feed-forward): [s], [s], [s][s] indexed [from][to] */
    int32_t q_rank, kv_rank;       /* sizes of the query latent and of the cached key/value latent */
    const float *q_lat_norm, *kv_lat_norm; /* [q_rank], [kv_rank] RMS norm weights of the latents */
    const void *w_uq;              /* [heads*dim][q_rank] */
    const void *w_uk_t;            /* [heads][kv_rank][dim]: per head the TRANSPOSED key up-projection: q_h is carried into the latent space */
    const void *w_uv;              /* [heads][vdim][kv_rank] */
    float *latent_pages;           /* [pages][page_size][kv_rank] */
    float gate_cap;                /* mLSTM: gate pre-activations z become cap tanh(z / cap) */
    float *rec_aux;                /* [slots][heads] running maxima of the stabilised recurrence (rec_state: [slots][heads][vdim + 1][dim]) */
    int32_t router;                /* lm_b200_router_kind */
    const float *router_bias;      /* [experts] added to the router logits; NULL: none */
    float act_limit, shared_limit; /* clamps of a CLAMPED_GLU: routed experts / dense unit, shared expert */

    /* ---- further mechanisms of the stream form (all zero / NULL where a record does not use them) ----
     * w_in of the mixers below, in this order:
     *   GATED_DELTA       q (kv_heads*dim) | k (kv_heads*dim) | v (heads*vdim) | beta (heads) | decay (heads) | gate (heads*vdim)
     *   RETENTION         q (heads*dim) | k (heads*dim) | v (heads*vdim) | gate (heads*vdim)
     *   LATENT_ATTENTION  query latent (q_rank) | key/value latent (kv_rank) | rotated key part (rot_dim) | gate (heads*vdim, unless GATE_NONE)
     * GATED_DELTA uses conv_taps, conv_w, conv_tail, a_log [heads], dt_bias [heads], unit_eps, head_norm [vdim] and rec_state
     * as CHANNEL_DELTA does; its decay is exp(-exp(a_log_h) softplus(z_h + dt_bias_h)) per head.  RETENTION: S <- head_decay_h S
     * + k v^T with k times dim^-1/2 after its rotation, o = S^T q, o / rms(o) per head (head_norm NULL: no weight).
     * FF_DENSE with ACT_RELU2: ws_gate_up holds the up rows alone [dense_ff][width]. */
    int32_t parallel;              /* != 0: the feed-forward reads the streams as they were BEFORE the mixer's write; both outputs are written at once */
    int32_t mixer_gate;            /* lm_b200_gate_kind */
    int32_t rot_layout;            /* lm_b200_rot_layout; RETENTION and LATENT_ATTENTION, with rot_dims / rot_freq as above */
    int32_t rot_dim;               /* LATENT_ATTENTION: every query head is [dim plain | rot_dim turned with the position]; ONE turned key part of
                                      this size, shared by all heads, is cached behind the latent: latent_pages [pages][page_size][kv_rank + rot_dim],
                                      w_uq [heads*(dim + rot_dim)][q_rank].  `window` > 0 limits its keys to the last `window` positions. */
    const float *head_decay;       /* [heads] RETENTION */
    int32_t identity_experts;      /* SOFTMAX_GROUPED: router outputs behind the `experts` real ones whose expert is the identity */
    int32_t group_count, group_keep; /* groups of neighbouring router outputs (experts + identity_experts must divide); <= 1 group: no restriction */
    float route_scale;             /* multiplies the normalised weights */
    const float *route_correction; /* [experts + identity_experts] added to the scores for the choice only; NULL: none */
    int32_t shared_gate;           /* != 0: w_router has one more row behind the router outputs, g; the shared unit's output is times sigmoid(g . h) */
} lm_b200_layer;

typedef struct lm_b200_model {
    int32_t n_layer, width, vocab, taps;             /* n_layer: layer records in execution order */
    int32_t page_size, max_pages, n_slots, max_rows; /* max_pages: per sequence; max_rows: rows of one forward call */
    float eps;                     /* inside the root of every RMS norm */
    int32_t precision;             /* lm_b200_precision */
    const void *embed, *head;      /* [vocab][width] */
    lm_b200_norm final_norm;
    const int32_t *page_table;     /* device, [n_slots][max_pages] */
    int32_t step_graphs;           /* != 0: steps of a few rows (decoding) replay a CUDA graph captured at their first use */
    float logit_scale;             /* multiplies the logits (0 is read as 1) */
    float embed_scale;             /* multiplies the embedding rows (0 is read as 1) */
    const float *embed_norm;       /* [width] RMS norm weight applied to the embedding rows (stream form); NULL: none */
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
/* a parallel record's mixer kernels alone on given stacked projections proj [M][n_in] (modified in place; state is
 * appended as in a step): out [M][heads * vdim], before the output projection */
int lm_b200_op_mixer_kernels(lm_b200_engine *e, int layer, float *proj, const int32_t *step, int M, int n_seq, float *out,
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

// lm_internal.h - shared declarations of the language-model path (lm_kernels.cu, lm_mixers.cu, lm_engine.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lm {

constexpr int kMaxTaps = 32;          // taps of the causal tap mix (the tail keeps taps - 1 rows per sequence)
constexpr int kRowsKernelMax = 8;     // up to this many rows a linear layer runs one warp per output element
constexpr int kRowsKernelMaxOut = 64; // ... and a linear layer of up to this many outputs at any number of rows
constexpr int kTileRows = 64;         // row tile of the tiled linear kernel = padding of an expert group on that kernel
constexpr int kAttnRowsKernelMax = 8; // up to this many rows attention splits every row's keys over CTAs
constexpr int kAttnSplitsMax = 32;    // most key splits of a row (sizes the partial-result workspace)

struct NormW { const float* w; const float* b; float alpha; };                  // DynamicTanh: tanh(alpha x) w + b
struct RowMeta { const int* slot; const int* pos; const int* start; };          // per row of the step
struct SeqMeta { const int* slot; const int* row0; const int* count; };         // per scheduled sequence
struct PageMap { const int* table; int max_pages; int page_size; };             // table[slot][max_pages] -> page
struct AttnShape {
    int heads, kv_heads, dim, window, keep_first;
    float scale, softcap;
    const float* temp; const float* slopes; const float* sink;                  // per query head; each may be null
};
// After a kernel of a short step gave x[a][n] its new value, the NEXT sublayer's input for that element can follow in the
// same thread when every scheduled sequence has exactly one row in the step: norm, taps over the sequence's tail, and
// the tail update are all per (sequence, channel).  h == nullptr: nothing follows.
struct TapOut {
    const float* nw; const float* nb; float alpha;   // the next sublayer's input norm
    const float* cw; int taps;                        // its taps [D][taps] (nullptr / 0: none)
    float* tail;                                      // its tail [slots][taps - 1][D]
    const int* row_slot; const int* row_pos;
    float* h;                                         // [M][D]
};
struct GroupMap { int* a_row; float* a_scale; int* a_expert; int* n_slots; };   // expert-grouped assignment slots
// Routing on the softmax over all n router outputs (n_real experts, then identity experts): choice on score + correction,
// restricted to the `keep` best of `count` groups of neighbours, weights = chosen scores / their sum x scale.  n == 0: not
// this rule.
struct GroupedRoute { int n; int n_real; int count; int keep; float scale; const float* correction; };
// activation of the gated units (kind: kGluSilu / kGluClamped of lm_device.cuh; the clamp of routed / dense and shared units)
struct GluAct { int kind; float limit; float shared_limit; };

cudaError_t launch_embed(const void* table_bf16, const int* ids, float* out, int M, int V, int D, cudaStream_t st);
cudaError_t launch_dyt_tapmix(const float* x, const NormW& n, const float* cw, int taps, const float* tail, const RowMeta& rm,
                              float* out, void* out_bf16, int M, int D, cudaStream_t st);
cudaError_t launch_tapmix_tail(const float* x, const NormW& n, int taps, float* tail, const SeqMeta& sm, int n_seq, int D,
                               cudaStream_t st);
cudaError_t launch_linear(const float* A, int lda, const void* W_bf16, long long w_expert_stride, float* Y, int ldy, int M,
                          int N, int K, const GroupMap* gm, cudaStream_t st);
// the fused forms for a step of at most kRowsKernelMax rows
cudaError_t launch_dyt_tapmix_seq(const float* x, const NormW& n, const float* cw, int taps, float* tail, const SeqMeta& sm,
                                  const RowMeta& rm, int n_seq, float* out, int D, cudaStream_t st);
cudaError_t launch_linear_rows_residual(const float* A, int lda, const void* W, float* x, int M, int N, int K, const NormW& n,
                                        const TapOut& next, cudaStream_t st);
cudaError_t launch_gated_rows(const float* A, int lda, const void* W, long long w_expert_stride, float* mid, int n_assign, int F,
                              int K, const GroupMap* gm, const void* Ws, float* smid, int n_shared_rows, int Sf, cudaStream_t st,
                              const GluAct& act = GluAct{0, 0.f, 0.f});
cudaError_t launch_down_combine_rows(const float* mid, int F, const void* Wd, const int* a_expert, int top, const float* smid,
                                     int Sf, const void* Wsd, float* x, int M, int D, const NormW& n, const TapOut& next,
                                     cudaStream_t st, const float* a_weight = nullptr, int n_real = 0, const float* ident_h = nullptr,
                                     const float* shared_gate = nullptr, int shared_gate_ld = 0);
cudaError_t launch_router_rows(const float* h, int D, const void* Wr, int E, int top, int M, float* z, const GroupMap& gm,
                               int* slot_of, cudaStream_t st, const float* bias = nullptr, bool softmax_top = false,
                               const GroupedRoute* gr = nullptr);
cudaError_t launch_qk_norm_cache(float* qk, int nq, int nk, const float* qw, const float* kw, float eps, float* kcache,
                                 float* vcache, const PageMap& pm, int kv_heads, int dim, const RowMeta& rm, int M,
                                 cudaStream_t st);
cudaError_t launch_sink_attention(const float* qk, int q_stride, const float* kcache, const float* vcache, const PageMap& pm,
                                  const AttnShape& a, const RowMeta& rm, float* out, void* out_bf16, float* split_ws,
                                  unsigned* arrived, int M, cudaStream_t st);
cudaError_t launch_router_topk(const float* z, int E, int top, int M, int* sel_e, float* sel_w, cudaStream_t st,
                               const float* bias = nullptr, bool softmax_top = false, const GroupedRoute* gr = nullptr);
cudaError_t launch_moe_group(const int* sel_e, const float* sel_w, int n_assign, int top, int E, int pad, const GroupMap& gm,
                             int* slot_of, int max_slots, cudaStream_t st);
cudaError_t launch_silu_mul(const float* gu, float* mid, void* mid_bf16, int M, int F, const GroupMap* gm, cudaStream_t st,
                            int act = 0, float limit = 0.f);
cudaError_t launch_pack_rows_bf16(const float* A, void* Ab, int M, int D, const GroupMap* gm, cudaStream_t st);
cudaError_t launch_residual_dyt(float* x, const float* y, const float* parts, const int* slot_of, int top, const NormW& n, int M,
                                int D, cudaStream_t st);
cudaError_t launch_dyt_gather(const float* x, const int* rows, const NormW& n, float* out, void* out_bf16, int M, int D,
                              cudaStream_t st);
cudaError_t launch_argmax_rows(const float* logits, int M, int V, int* out, cudaStream_t st);

// ---- the parallel layer form (lm_mixers.cu) ----
struct TalkShape {
    int heads, kv_heads, dim, vdim, rot_dims;
    float scale;
    const float* rot_freq;                                                      // [rot_dims / 2]
    const float* talk; const float* sink;                                       // [heads][heads], [heads]; each may be null
    int window;                                                                 // > 0: key j is seen from i only when i - j < window
};
struct DeltaShape {
    int heads, kv_heads, dim, vdim, taps;
    float unit_eps;
    const float* conv_w; const float* a_log; const float* dt_bias;
};
// columns of the recurrence's inputs in their row
struct ScanInputs { int q_off, k_off, a_off, v_off, beta_off; };

cudaError_t launch_layernorm_rows(const float* x, const int* rows, const float* w, const float* b, float eps, float out_scale,
                                  float* out, void* out_bf16, int M, int D, cudaStream_t st, bool rms = false);
cudaError_t launch_pair_rows(const float* x, const float* x0, float* cat, void* cat_bf16, int M, int D, cudaStream_t st);
cudaError_t launch_add_rows(float* x, const float* y, int M, int D, cudaStream_t st);
// relu2: max(z, 0)^2 instead of the xIELU; out may be null when only the bf16 copy is wanted
cudaError_t launch_xielu_rows(const float* proj, int ld, int off, float ap, float an, float* out, int ldo, int out_off,
                              void* out_bf16, int M, int F, cudaStream_t st, bool relu2 = false);
cudaError_t launch_talk_prep(float* proj, int ld, const float* bias, int q_off, int k_off, int v_off, int gate_off,
                             const TalkShape& a, const float* qw, const float* kw, float eps, float* kcache, float* vcache,
                             const PageMap& pm, const RowMeta& rm, int M, cudaStream_t st);
bool talk_attention_supported(const TalkShape& a);
cudaError_t launch_talk_attention(const float* proj, int ld, int q_off, int gate_off, const float* kcache, const float* vcache,
                                  const PageMap& pm, const TalkShape& a, const RowMeta& rm, float* out, int ldo, void* out_bf16,
                                  float* split_ws, unsigned* arrived, int M, cudaStream_t st);
// head_decay_off >= 0: ONE decay per head, exp(-exp(a_log_h) softplus(proj[head_decay_off + h] + dt_bias_h)); the rec row is
// then q | k | v | decay (H) | beta (H) and the output gate is left to the caller
cudaError_t launch_delta_prep(const float* proj, int ld, int beta_off, const DeltaShape& d, const float* tail, const RowMeta& rm,
                              float* rec, int ldr, int M, cudaStream_t st, int head_decay_off = -1);
cudaError_t launch_conv_tail(const float* proj, int ld, int C, int taps, float* tail, const SeqMeta& sm, int n_seq,
                             cudaStream_t st);
cudaError_t launch_gate_prep(float* proj, int ld, int q_off, int f_off, int v_off, const float* bias, const float* lower, int n_qf,
                             int n_v, int M, cudaStream_t st);
// early (both scans): launched so that it may start while its predecessor still runs (see launch_pdl_if)
cudaError_t launch_column_scan(const float* in, int ld, const ScanInputs& si, bool delta, int H, int G, int dim, int vdim,
                               float* state, const SeqMeta& sm, const RowMeta& rm, int n_seq, float* o, int ldo,
                               cudaStream_t st, bool head_decay = false, bool early = true);
// the same scan with scalar gates per (row, head): S <- a S + (b k) v^T and one more value column that is the constant 1
// (the normaliser n <- a n + b k, read out as n . q), so state and read-out have vdim + 1 columns per head.  a and b are
// columns a_off + h and beta_off + h of the input rows.  fixed_decay [H]: a = fixed_decay[h], b = 1 for every token instead.
// normaliser false: no extra column (state and read-out have vdim columns per head).
cudaError_t launch_scalar_gate_scan(const float* in, int ld, const ScanInputs& si, int H, int dim, int vdim, float* state,
                                    const SeqMeta& sm, const RowMeta& rm, int n_seq, float* o, int ldo, cudaStream_t st,
                                    const float* fixed_decay = nullptr, bool normaliser = true, bool early = true);
// gate_act: 0 the gate columns as they are, 1 their sigmoid, 2 their silu; w may be null (no weight)
cudaError_t launch_head_norm_gate(float* o, int ldo, void* o_bf16, const float* w, const float* gate, int ldg, int H, int vdim,
                                  float eps, int M, cudaStream_t st, int gate_act = 0);

// ---- the stream layer form (lm_streams.cu): hyper-connected residual streams, latent attention, stabilised matrix memory ----
// Per row: [x_j <- sum_s mix[s][j] x_s + out[j] (y + sum_t sel_w[t] parts[slot_of[t]])]  (y == nullptr and parts == nullptr:
// the streams stay), then u = sum_s in[s] x_s (in == nullptr: the plain sum) and h = layernorm(u) w (w == nullptr: h = u).
// rows (optional): the gathered rows h is wanted for (then nothing is written to the streams).
struct StreamWrite { const float* mix; const float* out; const float* y; const float* parts; const int* slot_of;
                     const float* sel_w; int top; };
// More of the same step: y2 / out2 - a second sublayer output written with its own weights (a record whose sublayers read
// the same streams); ident_h [M][D] - what an assignment without a slot (slot_of < 0, an identity expert) adds, times its
// weight; y_gate - y is multiplied by sigmoid(y_gate[row * y_gate_ld]); rms - the norm is x / sqrt(mean(x^2) + eps) w;
// norm_w2 / h2 / h2_b - a second norm weight on the same statistics and where its result goes.
struct StreamExtra { const float* y2; const float* out2; const float* ident_h; const float* y_gate; int y_gate_ld; int rms;
                     const float* norm_w2; float* h2; void* h2_b; };
cudaError_t launch_streams_step(float* X, int streams, const StreamWrite& wr, const float* in, const float* norm_w, float eps,
                                const int* rows, float* h, void* h_bf16, int M, int D, cudaStream_t st,
                                const StreamExtra& ex = StreamExtra{});
// norm_w: the rows get an RMS norm with this weight
cudaError_t launch_streams_embed(const void* table_bf16, const int* ids, float scale, float* X, int streams, int M, int V, int D,
                                 cudaStream_t st, const float* norm_w = nullptr, float eps = 0.f);
// n channels of which the first `dims` turn with the position (freq [dims / 2]; pairs (2i, 2i + 1), or (i, i + dims / 2) with
// half_layout)
struct RotPart { int n; int dims; int half_layout; const float* freq; };
// per row and head: dst[d_off + h dhs + c] = scale * turned(src[s_off + h shs + c]), c < n (rot.n is not read); heads below
// `split` take scale_a, the others scale_b
cudaError_t launch_rot_rows(const float* src, int lds, int s_off, int shs, float* dst, int ldd, int d_off, int dhs, int H, int n,
                            const RotPart& rot, int split, float scale_a, float scale_b, const RowMeta& rm, int M, cudaStream_t st);
// c_q = rms(proj[:, q_off : q_off + q_rank]) qw in place (+ its bf16 copy), c = rms(proj[:, c_off : c_off + kv_rank]) cw into
// the latent pages [page][page_size][kv_rank]
cudaError_t launch_latent_prep(float* proj, int ld, int q_off, int q_rank, int c_off, int kv_rank, const float* qw,
                               const float* cw, float eps, void* cq_bf16, float* pages, const PageMap& pm, const RowMeta& rm,
                               int M, cudaStream_t st, const RotPart& rot = RotPart{0, 0, 0, nullptr});
// attention of every (row, head) over the latent pages on its own (keys = values = the cached latents; q [M][H][R] carries
// the score multiplier): the fallback for shapes the tiled attention kernel does not take.  key_extra: page rows and queries
// have R + key_extra channels, all of them the key, the first R the value; window > 0: only the last `window` positions
bool latent_attention_rows_supported(int H, int R);
cudaError_t launch_latent_attention_rows(const float* q, const float* pages, const PageMap& pm, int H, int R, const float* sink,
                                         const RowMeta& rm, float* out, int M, cudaStream_t st, int key_extra = 0, int window = 0);
// Y[m][h N + n] = alpha * sum_k A[m][h K + k] W[h][n][k]  [* sigmoid(gate[m][h N + n])], fp32 arithmetic on bf16 weights.
// a_hs / y_hs > 0: the heads of A / Y are that many columns apart instead of K / N
cudaError_t launch_head_linear(const float* A, int lda, const void* W, float* Y, int ldy, void* y_bf16, int M, int H, int N, int K,
                               float alpha, const float* gate, int ldg, cudaStream_t st, int a_hs = 0, int y_hs = 0);
// log-space gates of the stabilised matrix memory, per (sequence, head) along the sequence's rows: i = cap tanh((z_i + b_i) /
// cap), f = logsigmoid(cap tanh((z_f + b_f) / cap)), m_t = max(f + m_(t-1), i) (m = 0 before position 0, carried in
// m_state[slot][head]); the columns i_off + h, f_off + h of the row become a = exp(f + m_(t-1) - m_t), b = exp(i - m_t), and
// floor_out[row][h] = exp(-m_t)
cudaError_t launch_mlstm_gates(float* proj, int ld, int i_off, int f_off, const float* bias, float cap, int H, float* m_state,
                               const SeqMeta& sm, const RowMeta& rm, int n_seq, float* floor_out, cudaStream_t st);
// o[r][h] = scale * raw[r][h][0:vdim] / (max(|scale * raw[r][h][vdim]|, floor[r][h]) + 1e-6), then / rms over the head, times
// w[h vdim + c] and sigmoid(gate[r][h vdim + c]); fp32 and the bf16 operand
cudaError_t launch_mlstm_finish(const float* raw, int ldr, const float* floor_in, float scale, const float* w, const float* gate,
                                int ldg, float eps, float* out, void* out_bf16, int M, int H, int vdim, cudaStream_t st);

}  // namespace lm

// lm_engine.cu - the C ABI of include/lm_b200.h: descriptor checks, the step workspace, and the launch sequence of one step.
//
// One step = embed, then per layer
//   h = tapmix(norm(x))                         dyt_tapmix (+ tail update)
//   [q | k] = h W_qk^T                          linear
//   q, k norms; k -> key pages, raw k -> value pages   qk_norm_cache
//   attention over the pages                    sink_attention
//   y = o W_o^T;  x += norm(y)                  linear, residual_dyt
//   h = tapmix'(norm'(x))                       dyt_tapmix (+ tail update)
//   z = h W_router^T; top experts; groups       linear, router_topk, moe_group
//   experts on score * h (grouped by expert)    linear (gate | up), silu_mul, linear (down)
//   the shared expert on h                      linear, silu_mul, linear
//   x += norm(shared + the row's expert rows)   residual_dyt
// and the final norm + head on the wanted rows.  Nothing here depends on how many sequences the rows belong to.
// A step of a few rows (decoding) runs the same arithmetic in fewer launches: norm + taps + tail in one, the output
// projection with the norm and residual add in its epilogue, router + top experts in one, the gate inside the gate | up
// product, and one kernel for the down products of a row's experts and the shared expert, their sum, the norm and the
// residual add.  When every sequence brings exactly one row (pure decoding), the kernels that finish a residual add
// also write the next sublayer's norm + taps and move its tail.
//
// A record of the parallel form (layer norm, one of the attention / recurrent mixers of lm_mixers.cu, a dense
// feed-forward) runs
//   [x = [x | x0] W_pre^T]                      pair_rows, linear            (x0: the embedding output; in front of a repeated block)
//   h = layernorm(x)                            layernorm_rows
//   proj = h W_in^T                             linear: every projection of the mixer and the feed-forward's up rows
//   mixer on proj -> out[:, :mixer columns]     talk_prep + talk_attention | gate_prep + column_scan + head_norm_gate |
//                                               linear x 2 (decay, gate) + delta_prep + conv_tail + column_scan + head_norm_gate
//   out[:, mixer columns:] = act(proj up rows)  xielu_rows
//   x += out W_out^T                            linear with the residual add (W_out = [W_o | W_down])
//
// A record of the stream form (s residual streams with hyper-connection weights, layer norm without bias, a latent
// attention or a stabilised matrix memory, a clamped gated unit or a mixture of them) runs, per sublayer,
//   x_j <- sum_s mix[s][j] x_s + out[j] y_prev;  h = layernorm(sum_s in[s] x_s)     streams_step: the previous sublayer's
//                                               write and this one's read in one launch
//   proj = h W_in^T                             linear: every projection that reads h
//   latent attention: latent norms, latent -> pages (latent_prep); q = c_q W_uq^T (linear); q_h -> q_h^T W_uk,h (head_linear);
//                     attention over the latent pages, all heads on the one latent "key/value head" (talk_attention);
//                     o_h = W_uv,h (attended latent) * sigmoid(gate) (head_linear)
//   matrix memory:    log-space gates and running maximum (mlstm_gates); the recurrence with the normaliser as one more
//                     value column (scalar_gate_scan); read-out / normaliser, head norm, gate (mlstm_finish)
//   y = out W_o^T                               linear
//   feed-forward:     [gate | up] product, clamped activation, down product; routed experts grouped as above, their outputs
//                     weighed by the softmax over the chosen logits inside the next streams_step
// and after the last layer the streams are summed for the final norm.  Norms of stream records are layer norms or RMS
// norms (x / sqrt(mean(x^2) + eps) w), the embedding output may pass an RMS norm of its own, and three more mixers stand
// beside the two above:
//   gated delta rule: convolutions, silu, unit norms, beta and ONE decay per head (delta_prep); tails (conv_tail); the
//                     recurrence (column_scan with a decay per head); per-head RMS norm x weight x silu(gate) (head_norm_gate)
//   retention:        q | k turned in place, k x dim^-1/2 (rot_rows); S <- decay_h S + k v^T, o = S^T q (scalar_gate_scan with a
//                     fixed decay, no normaliser); per-head RMS norm x silu(gate) (head_norm_gate)
//   latent attention with a turned key part and a window: the cached row is [latent | turned key part]; the latent-space
//                     query of a head is [q_plain^T W_uk | q_turned] (head_linear + rot_rows); the attention sees the last
//                     `window` rows
// A PARALLEL stream record lets both sublayers read the streams before either writes: the mixer's output waits in a buffer
// of its own, and one streams_step writes both outputs (and, with one stream, gave both sublayers their inputs: two norm
// weights on the same statistics).  The feed-forward may also be a dense squared-relu unit, and the mixture may route by
// the softmax over all router outputs with a choice correction, groups, identity experts (they add weight x input inside
// the next streams_step or down_combine_rows) and a sigmoid gate number on the shared unit (a column of the router logits).
//
// Products.  With float32 precision every product runs on the fp32 FMA kernels.  With bfloat16 precision a step of at
// least kTensorRowsMin rows (a prompt portion) runs its products on the tensor cores (the tcgen05 kernel of
// gemm_tcgen05.cu, bf16 operands, fp32 accumulation in tensor memory): the norm / attention / gate kernels write the
// bf16 operand beside their fp32 result, the expert groups are packed (gathered, scaled by the router score, padded to
// the 128-row tile) into one bf16 operand, and the output projection's epilogue applies the DynamicTanh and adds the
// residual stream.  Shorter steps (decoding) stream the weights once per row on the row kernels.  The router, norms,
// scores, softmax, pages and the residual stream are fp32 in both.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <map>
#include <new>
#include <tuple>
#include <vector>

#include <cuda_runtime.h>

#include "gemm_tcgen05.h"
#include "lm_b200.h"
#include "lm_internal.h"

namespace {

std::atomic<long long> g_launches{0};
thread_local char g_cuda_err[256] = "";

struct Guard {                                   // run on the engine's device, restore the caller's
    int prev = -1;
    bool ok = true;
    explicit Guard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~Guard() { if (prev >= 0) cudaSetDevice(prev); }
};

inline int cuda_fail(cudaError_t e) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return e == cudaErrorNotSupported ? LM_B200_EUNSUPPORTED : LM_B200_ECUDA;
}

#define LCK(call)                                       \
    do {                                                \
        cudaError_t e__ = (call);                       \
        if (e__ != cudaSuccess) return cuda_fail(e__);  \
        g_launches++;                                   \
    } while (0)

inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline lm::NormW N(const lm_b200_norm& n) { return lm::NormW{n.w, n.b, n.alpha}; }

}  // namespace

struct lm_b200_engine {
    lm_b200_model m;
    std::vector<lm_b200_layer> layers;
    int device = 0;
    char* arena = nullptr;
    size_t arena_bytes = 0;
    int max_slots = 0;                           // assignment slots of the widest expert layer
    // workspace (fp32 unless noted)
    float *x, *h, *qk, *att, *y, *z, *sel_w, *a_scale, *gu, *mid, *parts, *sgu, *smid, *hw;
    int *sel_e, *slot_of, *a_row, *a_expert, *n_slots;
    // bf16 operands of the tensor-core products (bfloat16 precision only)
    void *hb, *attb, *packb, *midb, *smidb, *hwb;
    // the parallel layer form: embedding output, [x | x0], stacked projections, recurrence inputs, [mixer out | ff act]
    float *x0, *cat, *proj, *rec, *outcat;
    void *catb, *outcatb;
    // the stream layer form: the streams [rows][s][width], query latents (bf16 operand), queries carried into the latent
    // space, attended latents / raw read-outs, normaliser floors, and two constants {0, 1}
    float *xs, *qlat, *olat, *floorb, *unit;
    void* cqb;
    // records whose sublayers read the same streams: the mixer's output beside the feed-forward's, and the feed-forward's input
    float *ymix, *h2;
    void* h2b;
    bool stream_form = false;
    float* split_ws;                             // partial results of the key splits of a few rows' attention
    unsigned* split_arrived;                     // ... and their arrival counters (zero between launches)
    // steps of a few rows are captured once per (rows, sequences, wanted) into a CUDA graph over these fixed buffers
    int32_t* step_static = nullptr;
    float* logits_static = nullptr;
    cudaStream_t capture_stream = nullptr;       // captures run here (the caller's stream may be the legacy default stream)
    struct StepGraph { cudaGraphExec_t exec; long long launches; };
    std::map<std::tuple<int, int, int>, StepGraph> graphs;
};

namespace {

constexpr int kTensorRowsMin = 32;               // rows of a step from which its products run on the tensor cores
constexpr int kHeadTensorRowsMin = 4;            // wanted rows from which the head does

// assignment slots of `rows` rows when every expert group is padded to `pad` slots
int slots_bound(int rows, int top, int experts, int pad) {
    const int n = rows * top;
    return n + std::min(experts, n) * (pad - 1);
}

bool tensor_path(const lm_b200_engine* e, int M, int N, int K) {
    return e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin && dia::gemm_tcgen05_shape_ok(M, N, K);
}

const dia::GemmEpilogue kPlain{nullptr, nullptr, nullptr, 0.f};

struct StepView {
    const int *token, *want;
    lm::RowMeta rm;
    lm::SeqMeta sm;
};
StepView view(const int32_t* step, int M, int n_seq) {
    StepView v;
    v.token = step;
    v.rm = lm::RowMeta{step + M, step + 2 * (size_t)M, step + 3 * (size_t)M};
    const int32_t* s = step + 4 * (size_t)M;
    v.sm = lm::SeqMeta{s, s + n_seq, s + 2 * (size_t)n_seq};
    v.want = s + 3 * (size_t)n_seq;
    return v;
}

// columns of the stacked projections of a parallel record
struct InCols { int q, k, v, gate, f, beta, a1, g1, up, n, mix_out; };
InCols in_cols(const lm_b200_layer& l) {
    InCols c{};
    const int H = l.heads, G = l.kv_heads, d = l.dim, dv = l.vdim;
    int at = 0;
    if (l.mixer == LM_B200_MIXER_TALK_ATTENTION) {
        c.q = at; at += H * d; c.k = at; at += G * d; c.v = at; at += G * dv; c.gate = at; at += H;
    } else if (l.mixer == LM_B200_MIXER_HGRN2) {
        c.q = at; at += H * d; c.f = at; at += H * d; c.v = at; at += H * dv;
    } else {
        c.q = at; at += G * d; c.k = at; at += G * d; c.v = at; at += H * dv; c.beta = at; at += H;
        c.a1 = at; at += l.rank_a; c.g1 = at; at += l.rank_g;
    }
    c.up = at;
    at += l.ff == LM_B200_FF_DENSE ? l.dense_ff : 0;
    c.n = (at + 3) & ~3;
    c.mix_out = H * dv;
    return c;
}
// row of the recurrence inputs of a channel delta record: q | k | v | decay | gate | beta
int rec_cols(const lm_b200_layer& l) {
    return l.mixer == LM_B200_MIXER_CHANNEL_DELTA ? 2 * l.kv_heads * l.dim + 2 * l.heads * l.vdim + l.heads * l.dim + l.heads : 0;
}
lm::TalkShape talk_shape(const lm_b200_layer& l) {
    return lm::TalkShape{l.heads, l.kv_heads, l.dim, l.vdim, l.rot_dims, l.scale, l.rot_freq, l.talk, l.sink};
}

int check_parallel_layer(const lm_b200_model& m, const lm_b200_layer& l) {
    if (l.norm_mix_in.kind != LM_B200_NORM_LAYER || !l.norm_mix_in.w || !l.norm_mix_in.b) return LM_B200_EINVAL;
    if (l.heads <= 0 || l.kv_heads <= 0 || l.heads % l.kv_heads || l.dim <= 0 || l.vdim <= 0 || l.dim > 256 || l.vdim > 65536)
        return LM_B200_EINVAL;
    if (!l.w_in || !l.w_out) return LM_B200_EINVAL;
    if (l.ff != LM_B200_FF_NONE && l.ff != LM_B200_FF_DENSE) return LM_B200_EUNSUPPORTED;
    if (l.ff == LM_B200_FF_DENSE && (l.dense_ff <= 0 || l.act != LM_B200_ACT_XIELU)) return LM_B200_EINVAL;
    const InCols c = in_cols(l);
    if (l.n_in != c.n || l.k_out != c.mix_out + (l.ff == LM_B200_FF_DENSE ? l.dense_ff : 0)) return LM_B200_EINVAL;
    switch (l.mixer) {
        case LM_B200_MIXER_TALK_ATTENTION:
            if (!l.q_norm || !l.k_norm || !l.k_pages || !l.v_pages || l.rot_dims < 0 || l.rot_dims % 2 || l.rot_dims > l.dim ||
                (l.rot_dims > 0 && !l.rot_freq))
                return LM_B200_EINVAL;
            if (!lm::talk_attention_supported(talk_shape(l))) return LM_B200_EUNSUPPORTED;
            return LM_B200_OK;
        case LM_B200_MIXER_HGRN2:
            if (l.heads != l.kv_heads || !l.head_norm || !l.rec_state) return LM_B200_EINVAL;
            return LM_B200_OK;
        case LM_B200_MIXER_CHANNEL_DELTA:
            if (!l.head_norm || !l.rec_state || !l.conv_w || !l.a_log || !l.dt_bias || !l.w_a2 || !l.w_g2 || l.rank_a <= 0 ||
                l.rank_g <= 0 || l.conv_taps < 1 || l.conv_taps > lm::kMaxTaps || (l.conv_taps > 1 && !l.conv_tail))
                return LM_B200_EINVAL;
            return LM_B200_OK;
        default: return LM_B200_EUNSUPPORTED;
    }
    (void)m;
}

// columns of the stacked projections of a stream record (gate < 0: the mixer has no gate columns)
struct StreamCols { int q, k, v, ig, fg, gate, lat_q, lat_c, beta, a, n; };
StreamCols stream_cols(const lm_b200_layer& l) {
    StreamCols c{};
    const int H = l.heads, G = l.kv_heads, d = l.dim, dv = l.vdim;
    int at = 0;
    if (l.mixer == LM_B200_MIXER_LATENT_ATTENTION) {
        c.lat_q = at; at += l.q_rank; c.lat_c = at; at += l.kv_rank + l.rot_dim;   // the latent, then the turned key part
    } else if (l.mixer == LM_B200_MIXER_GATED_DELTA) {
        c.q = at; at += G * d; c.k = at; at += G * d; c.v = at; at += H * dv; c.beta = at; at += H; c.a = at; at += H;
    } else if (l.mixer == LM_B200_MIXER_RETENTION) {
        c.q = at; at += H * d; c.k = at; at += H * d; c.v = at; at += H * dv;
    } else {
        c.q = at; at += H * d; c.k = at; at += H * d; c.v = at; at += H * dv; c.ig = at; at += H; c.fg = at; at += H;
    }
    c.gate = -1;
    if (l.mixer_gate != LM_B200_GATE_NONE) { c.gate = at; at += H * dv; }
    c.n = (at + 3) & ~3;
    return c;
}
// the attention over the cached rows [latent | turned key part]: all of a row is the key, its first kv_rank channels the value
lm::TalkShape latent_shape(const lm_b200_layer& l) {
    return lm::TalkShape{l.heads, 1, l.kv_rank + l.rot_dim, l.kv_rank, 0, 1.f, nullptr, nullptr, l.sink, l.window > 0 ? l.window : 0};
}
// row of the recurrence inputs of a gated delta record: q | k | v | decay | beta
int delta_rec_cols(const lm_b200_layer& l) {
    return l.mixer == LM_B200_MIXER_GATED_DELTA ? 2 * l.kv_heads * l.dim + l.heads * l.vdim + 2 * l.heads : 0;
}
bool stream_norm_ok(const lm_b200_norm& n) { return n.w && (n.kind == LM_B200_NORM_LAYER || n.kind == LM_B200_NORM_RMS); }
// router outputs of a record and the columns of its logits (the shared unit's gate row behind them)
int route_outputs(const lm_b200_layer& l) { return l.experts + (l.router == LM_B200_ROUTER_SOFTMAX_GROUPED ? l.identity_experts : 0); }
int route_cols(const lm_b200_layer& l) { return route_outputs(l) + (l.router == LM_B200_ROUTER_SOFTMAX_GROUPED && l.shared_gate ? 1 : 0); }

int check_stream_layer(const lm_b200_model& m, const lm_b200_layer& l) {
    if (l.streams < 1 || l.streams > 8) return LM_B200_EUNSUPPORTED;
    if (!stream_norm_ok(l.norm_mix_in)) return LM_B200_EINVAL;
    if (l.heads <= 0 || l.dim <= 0 || l.vdim <= 0 || !l.w_in || !l.w_o || l.n_in != stream_cols(l).n) return LM_B200_EINVAL;
    if (l.mixer_gate != LM_B200_GATE_SIGMOID && l.mixer_gate != LM_B200_GATE_NONE && l.mixer_gate != LM_B200_GATE_SILU)
        return LM_B200_EINVAL;
    for (int q = 0; q < (l.ff == LM_B200_FF_NONE ? 1 : 2); ++q)
        if (!l.hc_in[q] || !l.hc_out[q] || !l.hc_mix[q]) return LM_B200_EINVAL;
    const bool rot_ok = l.rot_dims >= 0 && l.rot_dims % 2 == 0 && (l.rot_dims == 0 || l.rot_freq) &&
                        (l.rot_layout == LM_B200_ROT_INTERLEAVED || l.rot_layout == LM_B200_ROT_HALF);
    switch (l.mixer) {
        case LM_B200_MIXER_LATENT_ATTENTION:
            if (l.q_rank <= 0 || l.kv_rank <= 0 || !l.q_lat_norm || !l.kv_lat_norm || !l.w_uq || !l.w_uk_t || !l.w_uv ||
                !l.latent_pages || l.rot_dim < 0 || !rot_ok || l.rot_dims > l.rot_dim)
                return LM_B200_EINVAL;
            if (l.mixer_gate == LM_B200_GATE_SILU) return LM_B200_EUNSUPPORTED;
            if (!lm::talk_attention_supported(latent_shape(l)) && !lm::latent_attention_rows_supported(l.heads, l.kv_rank + l.rot_dim))
                return LM_B200_EUNSUPPORTED;
            break;
        case LM_B200_MIXER_MLSTM:
            if (!l.head_norm || !l.rec_state || !l.rec_aux || !(l.gate_cap > 0.f) || l.mixer_gate != LM_B200_GATE_SIGMOID)
                return LM_B200_EINVAL;
            if (l.dim > 256 || l.heads > 65535) return LM_B200_EUNSUPPORTED;
            break;
        case LM_B200_MIXER_GATED_DELTA:
            if (l.kv_heads <= 0 || l.heads % l.kv_heads || !l.head_norm || !l.rec_state || !l.conv_w || !l.a_log || !l.dt_bias ||
                l.conv_taps < 1 || (l.conv_taps > 1 && !l.conv_tail))
                return LM_B200_EINVAL;
            if (l.dim > 256 || l.heads > 65535 || l.conv_taps > lm::kMaxTaps) return LM_B200_EUNSUPPORTED;
            break;
        case LM_B200_MIXER_RETENTION:
            if (!l.rec_state || !l.head_decay || !rot_ok || l.rot_dims > l.dim) return LM_B200_EINVAL;
            if (l.dim > 256 || l.heads > 32767) return LM_B200_EUNSUPPORTED;
            break;
        default: return LM_B200_EUNSUPPORTED;
    }
    if (l.ff == LM_B200_FF_NONE) return LM_B200_OK;
    if (!stream_norm_ok(l.norm_ff_in)) return LM_B200_EINVAL;
    if (l.parallel && l.norm_ff_in.kind != l.norm_mix_in.kind) return LM_B200_EUNSUPPORTED;
    if (l.ff == LM_B200_FF_DENSE && l.act == LM_B200_ACT_RELU2) return (l.dense_ff > 0 && l.ws_gate_up && l.ws_down) ? LM_B200_OK : LM_B200_EINVAL;
    if (l.act != LM_B200_ACT_CLAMPED_GLU && l.act != LM_B200_ACT_SILU_GLU) return LM_B200_EUNSUPPORTED;
    if (l.ff == LM_B200_FF_DENSE) return (l.dense_ff > 0 && l.ws_gate_up && l.ws_down) ? LM_B200_OK : LM_B200_EINVAL;
    if (l.ff != LM_B200_FF_ROUTED_EXPERTS) return LM_B200_EUNSUPPORTED;
    if (l.experts <= 0 || l.top <= 0 || l.expert_ff <= 0 || l.shared_ff < 0) return LM_B200_EINVAL;
    if (!l.w_router || !l.w_gate_up || !l.w_down || (l.shared_ff > 0 && (!l.ws_gate_up || !l.ws_down))) return LM_B200_EINVAL;
    if (l.router == LM_B200_ROUTER_SOFTMAX_GROUPED) {
        const int n = route_outputs(l);
        if (l.identity_experts < 0 || l.top > n || (l.shared_gate && l.shared_ff <= 0)) return LM_B200_EINVAL;
        if (l.group_count > 1 && (n % l.group_count || l.group_keep < 1 || l.group_keep > l.group_count ||
                                  l.top > l.group_keep * (n / l.group_count)))
            return LM_B200_EINVAL;
        if ((size_t)(2 * n + 1 + l.group_count) * sizeof(float) > 40000) return LM_B200_EUNSUPPORTED;
    } else if (l.router != LM_B200_ROUTER_SOFTMAX_TOP) {
        return LM_B200_EUNSUPPORTED;
    } else if (l.top > l.experts) {
        return LM_B200_EINVAL;
    }
    if (3 * (size_t)l.experts * sizeof(int) > 40000) return LM_B200_EUNSUPPORTED;
    (void)m;
    return LM_B200_OK;
}

int check_layer(const lm_b200_model& m, const lm_b200_layer& l) {
    if (l.form == LM_B200_FORM_PARALLEL) return check_parallel_layer(m, l);
    if (l.form == LM_B200_FORM_STREAMS) return check_stream_layer(m, l);
    if (l.form != LM_B200_FORM_SEQUENTIAL) return LM_B200_EUNSUPPORTED;
    if (l.mixer != LM_B200_MIXER_SINK_ATTENTION) return LM_B200_EUNSUPPORTED;
    if (l.heads <= 0 || l.kv_heads <= 0 || l.heads % l.kv_heads || l.dim <= 0 || l.dim > 256) return LM_B200_EINVAL;
    if (!l.w_qk || !l.q_norm || !l.k_norm || !l.w_o || !l.k_pages || !l.v_pages) return LM_B200_EINVAL;
    if (!l.norm_mix_in.w || !l.norm_mix_in.b || !l.norm_mix_out.w || !l.norm_mix_out.b) return LM_B200_EINVAL;
    if (m.taps > 1 && ((l.tap_mix && !l.tail_mix) || (l.tap_ff && !l.tail_ff))) return LM_B200_EINVAL;
    if (l.ff == LM_B200_FF_NONE) return LM_B200_OK;
    if (l.ff != LM_B200_FF_ROUTED_EXPERTS) return LM_B200_EUNSUPPORTED;
    if (l.experts <= 0 || l.top <= 0 || l.top > l.experts || l.expert_ff <= 0 || l.shared_ff < 0) return LM_B200_EINVAL;
    if (!l.w_router || !l.w_gate_up || !l.w_down || (l.shared_ff > 0 && (!l.ws_gate_up || !l.ws_down))) return LM_B200_EINVAL;
    if (!l.norm_ff_in.w || !l.norm_ff_in.b || !l.norm_ff_out.w || !l.norm_ff_out.b) return LM_B200_EINVAL;
    if (3 * (size_t)l.experts * sizeof(int) > 40000) return LM_B200_EUNSUPPORTED;
    return LM_B200_OK;
}

// the input of sublayer `sub` of layer l as something the previous kernel's epilogue can produce (lm::TapOut)
lm::TapOut tap_out(lm_b200_engine* e, const lm_b200_layer& l, int sub, const StepView& v) {
    const lm_b200_norm& n = sub ? l.norm_ff_in : l.norm_mix_in;
    const float* taps = sub ? l.tap_ff : l.tap_mix;
    return lm::TapOut{n.w, n.b, n.alpha, taps, taps ? e->m.taps : 0, sub ? l.tail_ff : l.tail_mix, v.rm.slot, v.rm.pos, e->h};
}

// h = tapmix(norm(x)) and the tail of every scheduled sequence
int norm_tapmix(lm_b200_engine* e, const lm_b200_layer& l, int sub, const float* x, const StepView& v, int M, int n_seq,
                float* out, cudaStream_t st) {
    const lm_b200_norm& n = sub ? l.norm_ff_in : l.norm_mix_in;
    const float* taps = sub ? l.tap_ff : l.tap_mix;
    float* tail = sub ? l.tail_ff : l.tail_mix;
    const int T = taps ? e->m.taps : 0;
    if (M <= lm::kRowsKernelMax) {                   // a few rows: norm, taps and the tail update in one launch
        LCK(lm::launch_dyt_tapmix_seq(x, N(n), taps, T, tail, v.sm, v.rm, n_seq, out, e->m.width, st));
        return LM_B200_OK;
    }
    void* out_b = (e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin && out == e->h) ? e->hb : nullptr;
    LCK(lm::launch_dyt_tapmix(x, N(n), taps, T, tail, v.rm, out, out_b, M, e->m.width, st));
    if (T > 1) LCK(lm::launch_tapmix_tail(x, N(n), T, tail, v.sm, n_seq, e->m.width, st));
    return LM_B200_OK;
}

// y = mixer(h); with fuse_x, x += norm_mix_out(y) instead (in the output projection's epilogue where that runs on the
// tensor cores).  hb: the bf16 copy of h when the caller has one.
int mixer(lm_b200_engine* e, const lm_b200_layer& l, const float* h, const void* hb, const StepView& v, int M, float* y,
          float* fuse_x, const lm::TapOut& next, cudaStream_t st) {
    const int D = e->m.width, nq = l.heads * l.dim, nk = l.kv_heads * l.dim;
    const lm::PageMap pm{e->m.page_table, e->m.max_pages, e->m.page_size};
    if (tensor_path(e, M, nq + nk, D)) {
        if (!hb) {
            LCK(lm::launch_pack_rows_bf16(h, e->hb, M, D, nullptr, st));
            hb = e->hb;
        }
        LCK(dia::launch_gemm_tcgen05_bf16(hb, 1, l.w_qk, nq + nk, e->qk, M, nq + nk, D, kPlain, nullptr, st));
    } else {
        LCK(lm::launch_linear(h, D, l.w_qk, 0, e->qk, nq + nk, M, nq + nk, D, nullptr, st));
    }
    LCK(lm::launch_qk_norm_cache(e->qk, nq, nk, l.q_norm, l.k_norm, e->m.eps, l.k_pages, l.v_pages, pm, l.kv_heads, l.dim,
                                 v.rm, M, st));
    const lm::AttnShape a{l.heads, l.kv_heads, l.dim, l.window, l.keep_first, l.scale, l.softcap, l.temp, l.slopes, l.sink};
    const bool tc_o = tensor_path(e, M, D, nq);
    LCK(lm::launch_sink_attention(e->qk, nq + nk, l.k_pages, l.v_pages, pm, a, v.rm, e->att, tc_o ? e->attb : nullptr, e->split_ws, e->split_arrived, M, st));
    if (tc_o) {
        if (fuse_x) {
            const dia::GemmEpilogue ep{fuse_x, l.norm_mix_out.w, l.norm_mix_out.b, l.norm_mix_out.alpha};
            LCK(dia::launch_gemm_tcgen05_bf16(e->attb, 1, l.w_o, D, fuse_x, M, D, nq, ep, nullptr, st));
            return LM_B200_OK;
        }
        LCK(dia::launch_gemm_tcgen05_bf16(e->attb, 1, l.w_o, D, y, M, D, nq, kPlain, nullptr, st));
    } else if (fuse_x && M <= lm::kRowsKernelMax) {
        LCK(lm::launch_linear_rows_residual(e->att, nq, l.w_o, fuse_x, M, D, nq, N(l.norm_mix_out), next, st));
        return LM_B200_OK;
    } else {
        LCK(lm::launch_linear(e->att, nq, l.w_o, 0, y, D, M, D, nq, nullptr, st));
    }
    if (fuse_x) LCK(lm::launch_residual_dyt(fuse_x, y, nullptr, nullptr, 0, N(l.norm_mix_out), M, D, st));
    return LM_B200_OK;
}

// x += norm(ff(h)) with a norm, x = ff(h) without.  A few rows: router + top experts + maps, gated products, and the
// sum over the row's experts with the norm and the residual add, four launches.  Longer steps group the (row, expert)
// assignments by expert for the tiled products.
int feed_forward(lm_b200_engine* e, const lm_b200_layer& l, const float* h, const void* hb, int M, float* x,
                 const lm_b200_norm* norm, const lm::TapOut& next, cudaStream_t st) {
    const int D = e->m.width, E = l.experts, top = l.top, F = l.expert_ff, Sf = l.shared_ff;
    const lm::NormW nrm = norm ? N(*norm) : lm::NormW{nullptr, nullptr, 0.f};
    if (M <= lm::kRowsKernelMax) {
        const lm::GroupMap rows{e->a_row, e->a_scale, e->a_expert, e->n_slots};
        LCK(lm::launch_router_rows(h, D, l.w_router, E, top, M, e->z, rows, e->slot_of, st));
        LCK(lm::launch_gated_rows(h, D, l.w_gate_up, 2LL * F * D, e->mid, M * top, F, D, &rows, l.ws_gate_up, e->smid,
                                  Sf > 0 ? M : 0, Sf, st));
        LCK(lm::launch_down_combine_rows(e->mid, F, l.w_down, e->a_expert, top, Sf > 0 ? e->smid : nullptr, Sf, l.ws_down, x, M, D,
                                         nrm, next, st));
        return LM_B200_OK;
    }
    LCK(lm::launch_linear(h, D, l.w_router, 0, e->z, E, M, E, D, nullptr, st));
    LCK(lm::launch_router_topk(e->z, E, top, M, e->sel_e, e->sel_w, st));
    const int n_assign = M * top;
    // both expert products on the tensor cores, or neither: the groups are padded to the row tile of the kernel that runs
    const bool tc = tensor_path(e, M, 2 * F, D) && tensor_path(e, M, D, F);
    const int pad = tc ? dia::kGemmRowTile : lm::kTileRows;
    const int bound = slots_bound(M, top, E, pad);
    const lm::GroupMap gm{e->a_row, e->a_scale, e->a_expert, e->n_slots};
    LCK(lm::launch_moe_group(e->sel_e, e->sel_w, n_assign, top, E, pad, gm, e->slot_of, bound, st));
    if (tc) {
        LCK(lm::launch_pack_rows_bf16(h, e->packb, bound, D, &gm, st));
        const dia::GemmGroups gu_groups{e->a_expert, 2 * F, e->n_slots}, down_groups{e->a_expert, D, e->n_slots};
        LCK(dia::launch_gemm_tcgen05_bf16(e->packb, 1, l.w_gate_up, (long long)E * 2 * F, e->gu, bound, 2 * F, D, kPlain,
                                          &gu_groups, st));
        LCK(lm::launch_silu_mul(e->gu, nullptr, e->midb, bound, F, &gm, st));
        LCK(dia::launch_gemm_tcgen05_bf16(e->midb, 1, l.w_down, (long long)E * D, e->parts, bound, D, F, kPlain, &down_groups, st));
    } else {
        LCK(lm::launch_linear(h, D, l.w_gate_up, 2LL * F * D, e->gu, 2 * F, bound, 2 * F, D, &gm, st));
        LCK(lm::launch_silu_mul(e->gu, e->mid, nullptr, bound, F, &gm, st));
        // the rows of mid are already in slot order: identity gather, no scale, the slots' experts
        const lm::GroupMap gm_down{nullptr, nullptr, e->a_expert, e->n_slots};
        LCK(lm::launch_linear(e->mid, F, l.w_down, (long long)D * F, e->parts, D, bound, D, F, &gm_down, st));
    }
    if (Sf > 0) {
        if (tensor_path(e, M, 2 * Sf, D) && tensor_path(e, M, D, Sf)) {
            if (!hb) {
                LCK(lm::launch_pack_rows_bf16(h, e->hb, M, D, nullptr, st));
                hb = e->hb;
            }
            LCK(dia::launch_gemm_tcgen05_bf16(hb, 1, l.ws_gate_up, 2 * Sf, e->sgu, M, 2 * Sf, D, kPlain, nullptr, st));
            LCK(lm::launch_silu_mul(e->sgu, nullptr, e->smidb, M, Sf, nullptr, st));
            LCK(dia::launch_gemm_tcgen05_bf16(e->smidb, 1, l.ws_down, D, e->y, M, D, Sf, kPlain, nullptr, st));
        } else {
            LCK(lm::launch_linear(h, D, l.ws_gate_up, 0, e->sgu, 2 * Sf, M, 2 * Sf, D, nullptr, st));
            LCK(lm::launch_silu_mul(e->sgu, e->smid, nullptr, M, Sf, nullptr, st));
            LCK(lm::launch_linear(e->smid, Sf, l.ws_down, 0, e->y, D, M, D, Sf, nullptr, st));
        }
    }
    LCK(lm::launch_residual_dyt(x, Sf > 0 ? e->y : nullptr, e->parts, e->slot_of, top, nrm, M, D, st));
    return LM_B200_OK;
}

// x = linear(A) or x += linear(A): the tensor-core kernel from kTensorRowsMin rows (its epilogue adds the residual),
// the row kernel for a few rows (likewise), the tiled fp32 kernel with a separate add in between
int product(lm_b200_engine* e, const float* A, const void* Ab, int lda, const void* W, float* out, int M, int N, int K,
            bool add, cudaStream_t st) {
    if (Ab && lda == K && tensor_path(e, M, N, K)) {
        const dia::GemmEpilogue ep{add ? out : nullptr, nullptr, nullptr, 0.f};
        LCK(dia::launch_gemm_tcgen05_bf16(Ab, 1, W, N, out, M, N, K, ep, nullptr, st));
        return LM_B200_OK;
    }
    if (!add) {
        LCK(lm::launch_linear(A, lda, W, 0, out, N, M, N, K, nullptr, st));
        return LM_B200_OK;
    }
    if (M <= lm::kRowsKernelMax) {
        LCK(lm::launch_linear_rows_residual(A, lda, W, out, M, N, K, lm::NormW{nullptr, nullptr, 0.f}, lm::TapOut{}, st));
        return LM_B200_OK;
    }
    LCK(lm::launch_linear(A, lda, W, 0, e->y, N, M, N, K, nullptr, st));
    LCK(lm::launch_add_rows(out, e->y, M, N, st));
    return LM_B200_OK;
}

// the mixer's own kernels on the stacked projections proj [M][c.n] (modified in place): the mixer's output lands in the
// first columns of e->outcat [M][k_out] (and its bf16 copy ob, if given)
int mixer_kernels(lm_b200_engine* e, const lm_b200_layer& l, const InCols& c, float* proj, const StepView& v, int M, int n_seq,
                  void* ob, cudaStream_t st) {
    const lm::PageMap pm{e->m.page_table, e->m.max_pages, e->m.page_size};
    const int ko = l.k_out;
    switch (l.mixer) {
        case LM_B200_MIXER_TALK_ATTENTION: {
            const lm::TalkShape a = talk_shape(l);
            LCK(lm::launch_talk_prep(proj, c.n, l.in_bias, c.q, c.k, c.v, c.gate, a, l.q_norm, l.k_norm, e->m.eps, l.k_pages,
                                     l.v_pages, pm, v.rm, M, st));
            LCK(lm::launch_talk_attention(proj, c.n, c.q, c.gate, l.k_pages, l.v_pages, pm, a, v.rm, e->outcat, ko, ob,
                                          e->split_ws, e->split_arrived, M, st));
            break;
        }
        case LM_B200_MIXER_HGRN2: {
            LCK(lm::launch_gate_prep(proj, c.n, c.q, c.f, c.v, l.in_bias, l.lower, l.heads * l.dim, l.heads * l.vdim, M, st));
            const lm::ScanInputs si{c.q, 0, c.f, c.v, 0};
            LCK(lm::launch_column_scan(proj, c.n, si, false, l.heads, l.heads, l.dim, l.vdim, l.rec_state, v.sm, v.rm, n_seq,
                                       e->outcat, ko, st, false, M <= lm::kRowsKernelMax));
            LCK(lm::launch_head_norm_gate(e->outcat, ko, ob, l.head_norm, nullptr, 0, l.heads, l.vdim, e->m.eps, M, st));
            break;
        }
        case LM_B200_MIXER_CHANNEL_DELTA: {
            const lm::DeltaShape d{l.heads, l.kv_heads, l.dim, l.vdim, l.conv_taps, l.unit_eps, l.conv_w, l.a_log, l.dt_bias};
            const int ldr = rec_cols(l), C = 2 * l.kv_heads * l.dim + l.heads * l.vdim;
            const int k0 = l.kv_heads * l.dim, v0 = 2 * k0, d0 = v0 + l.heads * l.vdim, g0 = d0 + l.heads * l.dim,
                      b0 = g0 + l.heads * l.vdim;
            // the second steps of the decay and gate projections: fp32 products (they enter the recurrence), straight into
            // the decay and gate columns of the recurrence inputs
            LCK(lm::launch_linear(proj + c.a1, c.n, l.w_a2, 0, e->rec + d0, ldr, M, l.heads * l.dim, l.rank_a, nullptr, st));
            LCK(lm::launch_linear(proj + c.g1, c.n, l.w_g2, 0, e->rec + g0, ldr, M, l.heads * l.vdim, l.rank_g, nullptr, st));
            LCK(lm::launch_delta_prep(proj, c.n, c.beta, d, l.conv_tail, v.rm, e->rec, ldr, M, st));
            LCK(lm::launch_conv_tail(proj, c.n, C, l.conv_taps, l.conv_tail, v.sm, n_seq, st));
            const lm::ScanInputs si{0, k0, d0, v0, b0};
            LCK(lm::launch_column_scan(e->rec, ldr, si, true, l.heads, l.kv_heads, l.dim, l.vdim, l.rec_state, v.sm, v.rm, n_seq,
                                       e->outcat, ko, st, false, M <= lm::kRowsKernelMax));
            LCK(lm::launch_head_norm_gate(e->outcat, ko, ob, l.head_norm, e->rec + g0, ldr, l.heads, l.vdim, e->m.eps, M, st));
            break;
        }
        default: return LM_B200_EUNSUPPORTED;
    }
    return LM_B200_OK;
}

// One record of the parallel form.  only == 0: x += mixer(h) + ff(h) with h = norm(x) (after the input mix, if the record
// has one).  only == 1 / 2: y = mixer(h_in) / ff(h_in) alone for a given h_in (operator boundaries).
int parallel_layer(lm_b200_engine* e, const lm_b200_layer& l, const StepView& v, int M, int n_seq, int only, const float* h_in,
                   float* y_out, cudaStream_t st) {
    const int D = e->m.width;
    const bool bf = e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin;
    const InCols c = in_cols(l);
    const float* h = h_in;
    const void* hb = nullptr;
    if (only == 0) {
        if (l.w_pre) {
            LCK(lm::launch_pair_rows(e->x, e->x0, e->cat, bf ? e->catb : nullptr, M, D, st));
            const int rc = product(e, e->cat, bf ? e->catb : nullptr, 2 * D, l.w_pre, e->x, M, D, 2 * D, false, st);
            if (rc) return rc;
        }
        LCK(lm::launch_layernorm_rows(e->x, nullptr, l.norm_mix_in.w, l.norm_mix_in.b, e->m.eps, 1.f, e->h, bf ? e->hb : nullptr, M,
                                      D, st));
        h = e->h;
        hb = bf ? e->hb : nullptr;
    } else if (bf) {
        LCK(lm::launch_pack_rows_bf16(h, e->hb, M, D, nullptr, st));
        hb = e->hb;
    }
    int rc = product(e, h, hb, D, l.w_in, e->proj, M, c.n, D, false, st);
    if (rc) return rc;
    const int ko = l.k_out;
    void* ob = bf ? e->outcatb : nullptr;
    if (only != 0) {
        if (cudaMemsetAsync(e->outcat, 0, (size_t)M * ko * 4, st) != cudaSuccess) return cuda_fail(cudaGetLastError());
        if (ob && cudaMemsetAsync(ob, 0, (size_t)M * ko * 2, st) != cudaSuccess) return cuda_fail(cudaGetLastError());
    }
    if (only != 2) {
        rc = mixer_kernels(e, l, c, e->proj, v, M, n_seq, ob, st);
        if (rc) return rc;
    }
    if (only != 1 && l.ff == LM_B200_FF_DENSE)
        LCK(lm::launch_xielu_rows(e->proj, c.n, c.up, l.act_p, l.act_q, e->outcat, ko, c.mix_out, ob, M, l.dense_ff, st));
    return product(e, e->outcat, ob, ko, l.w_out, only == 0 ? e->x : y_out, M, D, ko, only == 0, st);
}

// ---- the stream form ----------------------------------------------------------------------------------------------------
// Y = A W^T for an operand that has a contiguous bf16 copy Ab [M][K] (tensor cores) or lives in fp32 rows of stride lda
int product_ld(lm_b200_engine* e, const float* A, int lda, const void* Ab, const void* W, float* out, int M, int N, int K,
               cudaStream_t st) {
    if (Ab && tensor_path(e, M, N, K)) {
        LCK(dia::launch_gemm_tcgen05_bf16(Ab, 1, W, N, out, M, N, K, kPlain, nullptr, st));
        return LM_B200_OK;
    }
    LCK(lm::launch_linear(A, lda, W, 0, out, N, M, N, K, nullptr, st));
    return LM_B200_OK;
}

// y = mixer(h) of a stream record
int stream_mixer(lm_b200_engine* e, const lm_b200_layer& l, const float* h, const void* hb, const StepView& v, int M, int n_seq,
                 float* y, cudaStream_t st) {
    const int D = e->m.width, H = l.heads, nv = H * l.vdim;
    const bool bf = e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin;
    const StreamCols c = stream_cols(l);
    int rc = product_ld(e, h, D, hb, l.w_in, e->proj, M, c.n, D, st);
    if (rc) return rc;
    const float* gate = c.gate >= 0 ? e->proj + c.gate : nullptr;
    const int gate_act = l.mixer_gate == LM_B200_GATE_SILU ? 2 : 1;
    if (l.mixer == LM_B200_MIXER_LATENT_ATTENTION) {
        const lm::PageMap pm{e->m.page_table, e->m.max_pages, e->m.page_size};
        // a query head is [dim plain | rot_dim turned]; a cached row is [latent | turned key part]
        const int rd = l.rot_dim, dq = l.dim + rd, RK = l.kv_rank + rd, nq = H * dq, nl = H * RK, no = H * l.kv_rank;
        const lm::RotPart rot{rd, l.rot_dims, l.rot_layout, l.rot_freq};
        LCK(lm::launch_latent_prep(e->proj, c.n, c.lat_q, l.q_rank, c.lat_c, l.kv_rank, l.q_lat_norm, l.kv_lat_norm, e->m.eps,
                                   bf ? e->cqb : nullptr, l.latent_pages, pm, v.rm, M, st, rot));
        rc = product_ld(e, e->proj + c.lat_q, c.n, bf ? e->cqb : nullptr, l.w_uq, e->qk, M, nq, l.q_rank, st);
        if (rc) return rc;
        // scores q_h . (W_uk,h c_j) = (W_uk,h^T q_h) . c_j: the query goes into the latent space, with the score multiplier;
        // its turned part stands behind it, against the turned key part of the cached row
        LCK(lm::launch_head_linear(e->qk, nq, l.w_uk_t, e->qlat, nl, nullptr, M, H, l.kv_rank, l.dim, l.scale, nullptr, 0, st, dq, RK));
        if (rd > 0)
            LCK(lm::launch_rot_rows(e->qk, nq, l.dim, dq, e->qlat, nl, l.kv_rank, RK, H, rd, rot, H, l.scale, l.scale, v.rm, M, st));
        if (lm::talk_attention_supported(latent_shape(l)))
            LCK(lm::launch_talk_attention(e->qlat, nl, 0, -1, l.latent_pages, l.latent_pages, pm, latent_shape(l), v.rm, e->olat, no,
                                          nullptr, e->split_ws, e->split_arrived, M, st));
        else
            LCK(lm::launch_latent_attention_rows(e->qlat, l.latent_pages, pm, H, l.kv_rank, l.sink, v.rm, e->olat, M, st, rd,
                                                 l.window > 0 ? l.window : 0));
        // sum_j p_j (W_uv,h c_j) = W_uv,h (sum_j p_j c_j), times the sigmoid of the gate columns
        LCK(lm::launch_head_linear(e->olat, no, l.w_uv, e->att, nv, bf ? e->attb : nullptr, M, H, l.vdim, l.kv_rank, 1.f, gate, c.n, st));
    } else if (l.mixer == LM_B200_MIXER_GATED_DELTA) {
        const lm::DeltaShape d{H, l.kv_heads, l.dim, l.vdim, l.conv_taps, l.unit_eps, l.conv_w, l.a_log, l.dt_bias};
        const int k0 = l.kv_heads * l.dim, v0 = 2 * k0, d0 = v0 + nv, b0 = d0 + H, ldr = delta_rec_cols(l);
        LCK(lm::launch_delta_prep(e->proj, c.n, c.beta, d, l.conv_tail, v.rm, e->rec, ldr, M, st, c.a));
        LCK(lm::launch_conv_tail(e->proj, c.n, v0 + nv, l.conv_taps, l.conv_tail, v.sm, n_seq, st));
        const lm::ScanInputs si{0, k0, d0, v0, b0};
        LCK(lm::launch_column_scan(e->rec, ldr, si, true, H, l.kv_heads, l.dim, l.vdim, l.rec_state, v.sm, v.rm, n_seq, e->att, nv, st,
                                   true, M <= lm::kRowsKernelMax));
        LCK(lm::launch_head_norm_gate(e->att, nv, bf ? e->attb : nullptr, l.head_norm, gate, c.n, H, l.vdim, e->m.eps, M, st, gate_act));
    } else if (l.mixer == LM_B200_MIXER_RETENTION) {
        // q and k (adjacent in the row) turn in place, k also takes dim^-1/2; decay fixed per head, no write gate, no normaliser
        const lm::RotPart rot{l.dim, l.rot_dims, l.rot_layout, l.rot_freq};
        LCK(lm::launch_rot_rows(e->proj, c.n, c.q, l.dim, e->proj, c.n, c.q, l.dim, 2 * H, l.dim, rot, H, 1.f,
                                1.0f / sqrtf((float)l.dim), v.rm, M, st));
        const lm::ScanInputs si{c.q, c.k, 0, c.v, 0};
        LCK(lm::launch_scalar_gate_scan(e->proj, c.n, si, H, l.dim, l.vdim, l.rec_state, v.sm, v.rm, n_seq, e->att, nv, st,
                                        l.head_decay, false, M <= lm::kRowsKernelMax));
        LCK(lm::launch_head_norm_gate(e->att, nv, bf ? e->attb : nullptr, l.head_norm, gate, c.n, H, l.vdim, e->m.eps, M, st, gate_act));
    } else {
        LCK(lm::launch_mlstm_gates(e->proj, c.n, c.ig, c.fg, l.in_bias, l.gate_cap, H, l.rec_aux, v.sm, v.rm, n_seq, e->floorb, st));
        const lm::ScanInputs si{c.q, c.k, c.fg, c.v, c.ig};      // decay in the forget column, write strength in the input column
        LCK(lm::launch_scalar_gate_scan(e->proj, c.n, si, H, l.dim, l.vdim, l.rec_state, v.sm, v.rm, n_seq, e->olat,
                                        H * (l.vdim + 1), st, nullptr, true, M <= lm::kRowsKernelMax));
        LCK(lm::launch_mlstm_finish(e->olat, H * (l.vdim + 1), e->floorb, 1.0f / sqrtf((float)l.dim), l.head_norm, e->proj + c.gate,
                                    c.n, e->m.eps, e->att, bf ? e->attb : nullptr, M, H, l.vdim, st));
    }
    return product_ld(e, e->att, nv, bf ? e->attb : nullptr, l.w_o, y, M, D, nv, st);
}

// a dense unit that is not gated: out = max(h W_up^T, 0)^2 W_down^T
int relu2_unit(lm_b200_engine* e, const float* h, const void* hb, int M, const void* w_up, const void* w_down, int F, float* out,
               cudaStream_t st) {
    const int D = e->m.width;
    if (hb && tensor_path(e, M, F, D) && tensor_path(e, M, D, F)) {
        LCK(dia::launch_gemm_tcgen05_bf16(hb, 1, w_up, F, e->sgu, M, F, D, kPlain, nullptr, st));
        LCK(lm::launch_xielu_rows(e->sgu, F, 0, 0.f, 0.f, nullptr, F, 0, e->smidb, M, F, st, true));
        LCK(dia::launch_gemm_tcgen05_bf16(e->smidb, 1, w_down, D, out, M, D, F, kPlain, nullptr, st));
        return LM_B200_OK;
    }
    LCK(lm::launch_linear(h, D, w_up, 0, e->sgu, F, M, F, D, nullptr, st));
    LCK(lm::launch_xielu_rows(e->sgu, F, 0, 0.f, 0.f, e->smid, F, 0, nullptr, M, F, st, true));
    LCK(lm::launch_linear(e->smid, F, w_down, 0, out, D, M, D, F, nullptr, st));
    return LM_B200_OK;
}

// one gated unit on all rows: out = act([gate | up] h) W_down^T
int gated_unit(lm_b200_engine* e, const lm_b200_layer& l, const float* h, const void* hb, int M, const void* w_gu, const void* w_down,
               int F, float limit, float* out, cudaStream_t st) {
    const int D = e->m.width;
    if (hb && tensor_path(e, M, 2 * F, D) && tensor_path(e, M, D, F)) {
        LCK(dia::launch_gemm_tcgen05_bf16(hb, 1, w_gu, 2 * F, e->sgu, M, 2 * F, D, kPlain, nullptr, st));
        LCK(lm::launch_silu_mul(e->sgu, nullptr, e->smidb, M, F, nullptr, st, l.act == LM_B200_ACT_CLAMPED_GLU ? 1 : 0, limit));
        LCK(dia::launch_gemm_tcgen05_bf16(e->smidb, 1, w_down, D, out, M, D, F, kPlain, nullptr, st));
        return LM_B200_OK;
    }
    if (M <= lm::kRowsKernelMax) {                              // the gate inside the [gate | up] product
        const lm::GluAct act{l.act == LM_B200_ACT_CLAMPED_GLU ? 1 : 0, limit, limit};
        LCK(lm::launch_gated_rows(h, D, nullptr, 0, nullptr, 0, F, D, nullptr, w_gu, e->smid, M, F, st, act));
    } else {
        LCK(lm::launch_linear(h, D, w_gu, 0, e->sgu, 2 * F, M, 2 * F, D, nullptr, st));
        LCK(lm::launch_silu_mul(e->sgu, e->smid, nullptr, M, F, nullptr, st, l.act == LM_B200_ACT_CLAMPED_GLU ? 1 : 0, limit));
    }
    LCK(lm::launch_linear(e->smid, F, w_down, 0, out, D, M, D, F, nullptr, st));
    return LM_B200_OK;
}

// the feed-forward of a stream record: fills what the following streams_step adds (wr->y and, for grouped experts, the
// expert outputs with their weights; wx: the input rows identity experts return, the shared unit's gate)
int stream_ff(lm_b200_engine* e, const lm_b200_layer& l, const float* h, const void* hb, int M, lm::StreamWrite* wr,
              lm::StreamExtra* wx, cudaStream_t st) {
    const int D = e->m.width, E = l.experts, top = l.top, F = l.expert_ff, Sf = l.shared_ff;
    const int act = l.act == LM_B200_ACT_CLAMPED_GLU ? 1 : 0;
    wr->y = e->y; wr->parts = nullptr; wr->slot_of = nullptr; wr->sel_w = nullptr; wr->top = 0;
    if (l.ff == LM_B200_FF_DENSE) {
        if (l.act == LM_B200_ACT_RELU2) return relu2_unit(e, h, hb, M, l.ws_gate_up, l.ws_down, l.dense_ff, e->y, st);
        return gated_unit(e, l, h, hb, M, l.ws_gate_up, l.ws_down, l.dense_ff, l.act_limit, e->y, st);
    }
    const bool grouped = l.router == LM_B200_ROUTER_SOFTMAX_GROUPED;
    const int Et = route_outputs(l), zc = route_cols(l);         // router outputs; columns of the logits (+ the shared unit's gate)
    const lm::GroupedRoute gr{Et, E, l.group_count, l.group_keep, l.route_scale, l.route_correction};
    const float* sgate = (grouped && l.shared_gate) ? e->z + Et : nullptr;
    if (M <= lm::kRowsKernelMax) {
        const lm::GroupMap rows{e->a_row, e->a_scale, e->a_expert, e->n_slots};
        LCK(lm::launch_router_rows(h, D, l.w_router, zc, top, M, e->z, rows, e->slot_of, st, l.router_bias, !grouped,
                                   grouped ? &gr : nullptr));
        const lm::GroupMap unscaled{e->a_row, nullptr, e->a_expert, e->n_slots};    // the weight is for the expert's OUTPUT
        const lm::GluAct ga{act, l.act_limit, l.shared_limit};
        LCK(lm::launch_gated_rows(h, D, l.w_gate_up, 2LL * F * D, e->mid, M * top, F, D, &unscaled, l.ws_gate_up, e->smid,
                                  Sf > 0 ? M : 0, Sf, st, ga));
        LCK(lm::launch_down_combine_rows(e->mid, F, l.w_down, e->a_expert, top, Sf > 0 ? e->smid : nullptr, Sf, l.ws_down, e->y, M, D,
                                         lm::NormW{nullptr, nullptr, 0.f}, lm::TapOut{}, st, e->a_scale, grouped ? E : 0,
                                         grouped ? h : nullptr, sgate, zc));
        return LM_B200_OK;
    }
    LCK(lm::launch_linear(h, D, l.w_router, 0, e->z, zc, M, zc, D, nullptr, st));
    LCK(lm::launch_router_topk(e->z, zc, top, M, e->sel_e, e->sel_w, st, l.router_bias, !grouped, grouped ? &gr : nullptr));
    const bool tc = hb && tensor_path(e, M, 2 * F, D) && tensor_path(e, M, D, F);
    const int pad = tc ? dia::kGemmRowTile : lm::kTileRows;
    const int bound = slots_bound(M, top, E, pad);
    const lm::GroupMap gm{e->a_row, e->a_scale, e->a_expert, e->n_slots};
    const lm::GroupMap gather{e->a_row, nullptr, e->a_expert, e->n_slots};
    LCK(lm::launch_moe_group(e->sel_e, e->sel_w, M * top, top, E, pad, gm, e->slot_of, bound, st));
    if (tc) {
        LCK(lm::launch_pack_rows_bf16(h, e->packb, bound, D, &gather, st));
        const dia::GemmGroups gu_groups{e->a_expert, 2 * F, e->n_slots}, down_groups{e->a_expert, D, e->n_slots};
        LCK(dia::launch_gemm_tcgen05_bf16(e->packb, 1, l.w_gate_up, (long long)E * 2 * F, e->gu, bound, 2 * F, D, kPlain,
                                          &gu_groups, st));
        LCK(lm::launch_silu_mul(e->gu, nullptr, e->midb, bound, F, &gm, st, act, l.act_limit));
        LCK(dia::launch_gemm_tcgen05_bf16(e->midb, 1, l.w_down, (long long)E * D, e->parts, bound, D, F, kPlain, &down_groups, st));
    } else {
        LCK(lm::launch_linear(h, D, l.w_gate_up, 2LL * F * D, e->gu, 2 * F, bound, 2 * F, D, &gather, st));
        LCK(lm::launch_silu_mul(e->gu, e->mid, nullptr, bound, F, &gm, st, act, l.act_limit));
        const lm::GroupMap gm_down{nullptr, nullptr, e->a_expert, e->n_slots};
        LCK(lm::launch_linear(e->mid, F, l.w_down, (long long)D * F, e->parts, D, bound, D, F, &gm_down, st));
    }
    wr->y = nullptr;
    if (Sf > 0) {
        const int rc = gated_unit(e, l, h, hb, M, l.ws_gate_up, l.ws_down, Sf, l.shared_limit, e->y, st);
        if (rc) return rc;
        wr->y = e->y;
        wx->y_gate = sgate;
        wx->y_gate_ld = zc;
    }
    wr->parts = e->parts; wr->slot_of = e->slot_of; wr->sel_w = e->sel_w; wr->top = top;
    if (grouped) wx->ident_h = h;
    return LM_B200_OK;
}

}  // namespace

extern "C" {

int lm_b200_abi_version(void) { return LM_B200_ABI_VERSION; }
const char* lm_b200_last_cuda_error(void) { return g_cuda_err; }
int64_t lm_b200_launch_count(void) { return g_launches.load(); }

int lm_b200_engine_create(const lm_b200_model* model, const lm_b200_layer* layers, int device, lm_b200_engine** out) {
    if (!model || !layers || !out) return LM_B200_EINVAL;
    const lm_b200_model& m = *model;
    if (m.n_layer <= 0 || m.width <= 0 || m.vocab <= 0 || m.taps < 0 || m.taps > lm::kMaxTaps || m.page_size <= 0 ||
        m.max_pages <= 0 || m.n_slots <= 0 || m.max_rows <= 0 ||
        (m.precision != LM_B200_PRECISION_FP32 && m.precision != LM_B200_PRECISION_BF16) || !m.embed || !m.head || !m.final_norm.w ||
        (!m.final_norm.b && m.final_norm.kind != LM_B200_NORM_LAYER && m.final_norm.kind != LM_B200_NORM_RMS) || !m.page_table)
        return LM_B200_EINVAL;
    for (int i = 0; i < m.n_layer; ++i) {
        const int rc = check_layer(m, layers[i]);
        if (rc != LM_B200_OK) return rc;
        // the streams run through the whole stack: a stream record stands among stream records with the same number of them
        if ((layers[i].form == LM_B200_FORM_STREAMS) != (layers[0].form == LM_B200_FORM_STREAMS)) return LM_B200_EUNSUPPORTED;
        if (layers[i].form == LM_B200_FORM_STREAMS && layers[i].streams != layers[0].streams) return LM_B200_EINVAL;
    }
    Guard g(device);
    if (!g.ok) return LM_B200_ECUDA;
    lm_b200_engine* e = new (std::nothrow) lm_b200_engine();
    if (!e) return LM_B200_ENOMEM;
    e->m = m;
    e->layers.assign(layers, layers + m.n_layer);
    e->device = device;
    const size_t R = (size_t)m.max_rows, D = (size_t)m.width;
    size_t qk = 0, att = 0, E = 1, top = 1, F = 1, Sf = 1, slots = 1;
    size_t n_in = 0, k_out = 0, n_rec = 0, split_dim = 0;
    size_t n_streams = 0, n_lat = 0, q_rank = 0, n_heads = 0;
    bool pre = false, any_parallel = false;
    e->stream_form = e->layers[0].form == LM_B200_FORM_STREAMS;
    for (const lm_b200_layer& l : e->layers) {
        if (l.form == LM_B200_FORM_STREAMS) {
            n_streams = (size_t)l.streams;
            n_in = std::max(n_in, (size_t)l.n_in);
            att = std::max(att, (size_t)l.heads * l.vdim);
            n_heads = std::max(n_heads, (size_t)l.heads);
            if (l.mixer == LM_B200_MIXER_LATENT_ATTENTION) {
                qk = std::max(qk, (size_t)l.heads * (l.dim + l.rot_dim));
                n_lat = std::max(n_lat, (size_t)l.heads * (l.kv_rank + l.rot_dim));
                q_rank = std::max(q_rank, (size_t)l.q_rank);
                if (lm::talk_attention_supported(latent_shape(l))) split_dim = std::max(split_dim, (size_t)l.heads * (l.kv_rank + 2));
            } else if (l.mixer == LM_B200_MIXER_MLSTM) {
                n_lat = std::max(n_lat, (size_t)l.heads * (l.vdim + 1));
            }
            n_rec = std::max(n_rec, (size_t)delta_rec_cols(l));
            any_parallel = any_parallel || (l.parallel && l.ff != LM_B200_FF_NONE);
            if (l.ff == LM_B200_FF_DENSE) Sf = std::max(Sf, (size_t)l.dense_ff);
            if (l.ff == LM_B200_FF_ROUTED_EXPERTS) {
                E = std::max(E, (size_t)route_cols(l));
                top = std::max(top, (size_t)l.top);
                F = std::max(F, (size_t)l.expert_ff);
                Sf = std::max(Sf, (size_t)l.shared_ff);
                slots = std::max(slots, (size_t)slots_bound(m.max_rows, l.top, l.experts, dia::kGemmRowTile));
            }
            continue;
        }
        if (l.form == LM_B200_FORM_PARALLEL) {
            n_in = std::max(n_in, (size_t)l.n_in);
            k_out = std::max(k_out, (size_t)l.k_out);
            n_rec = std::max(n_rec, (size_t)rec_cols(l));
            pre = pre || l.w_pre;
            if (l.mixer == LM_B200_MIXER_TALK_ATTENTION) split_dim = std::max(split_dim, (size_t)l.heads * (l.vdim + 2));
            continue;
        }
        qk = std::max(qk, (size_t)(l.heads + l.kv_heads) * l.dim);
        att = std::max(att, (size_t)l.heads * l.dim);
        split_dim = std::max(split_dim, (size_t)l.heads * (l.dim + 2));
        if (l.ff == LM_B200_FF_ROUTED_EXPERTS) {
            E = std::max(E, (size_t)l.experts);
            top = std::max(top, (size_t)l.top);
            F = std::max(F, (size_t)l.expert_ff);
            Sf = std::max(Sf, (size_t)l.shared_ff);
            slots = std::max(slots, (size_t)slots_bound(m.max_rows, l.top, l.experts, dia::kGemmRowTile));
        }
    }
    e->max_slots = (int)slots;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t at = off; off += (bytes + 255) & ~(size_t)255; return at; };
    const size_t o_x = take(R * D * 4), o_h = take(R * D * 4), o_qk = take(R * qk * 4), o_att = take(R * att * 4),
                 o_y = take(R * D * 4), o_z = take(R * E * 4), o_sel_w = take(R * top * 4), o_sel_e = take(R * top * 4),
                 o_slot_of = take(R * top * 4), o_a_row = take(slots * 4), o_a_scale = take(slots * 4),
                 o_a_expert = take(slots * 4), o_n_slots = take(4), o_gu = take(slots * 2 * F * 4), o_mid = take(slots * F * 4),
                 o_parts = take(slots * D * 4), o_sgu = take(R * 2 * Sf * 4), o_smid = take(R * Sf * 4), o_hw = take(R * D * 4);
    const size_t o_x0 = take(pre ? R * D * 4 : 0), o_cat = take(pre ? R * 2 * D * 4 : 0), o_proj = take(R * n_in * 4),
                 o_rec = take(R * n_rec * 4), o_outcat = take(R * k_out * 4);
    const size_t o_xs = take(R * n_streams * D * 4), o_qlat = take(R * n_lat * 4), o_olat = take(R * n_lat * 4),
                 o_floor = take(R * n_heads * 4), o_unit = take(2 * 4);
    const size_t o_ymix = take(any_parallel ? R * D * 4 : 0), o_h2 = take(any_parallel ? R * D * 4 : 0);
    const size_t o_split = take((size_t)lm::kAttnRowsKernelMax * lm::kAttnSplitsMax * split_dim * 4);
    size_t max_heads = 1;
    for (const lm_b200_layer& l : e->layers) max_heads = std::max(max_heads, (size_t)l.heads);
    const size_t arrived_bytes = (size_t)lm::kAttnRowsKernelMax * max_heads * 4, o_arrived = take(arrived_bytes);
    const size_t o_step = take((size_t)(8 * lm::kRowsKernelMax) * 4), o_logits = take((size_t)lm::kRowsKernelMax * m.vocab * 4);
    const bool tcb = m.precision == LM_B200_PRECISION_BF16;
    const size_t o_hb = take(tcb ? R * D * 2 : 0), o_attb = take(tcb ? R * att * 2 : 0), o_packb = take(tcb ? slots * D * 2 : 0),
                 o_midb = take(tcb ? slots * F * 2 : 0), o_smidb = take(tcb ? R * Sf * 2 : 0), o_hwb = take(tcb ? R * D * 2 : 0);
    const size_t o_catb = take(tcb && pre ? R * 2 * D * 2 : 0), o_outcatb = take(tcb ? R * k_out * 2 : 0);
    const size_t o_cqb = take(tcb ? R * q_rank * 2 : 0), o_h2b = take(tcb && any_parallel ? R * D * 2 : 0);
    if (cudaMalloc(&e->arena, off) != cudaSuccess) {
        (void)cudaGetLastError();
        delete e;
        return LM_B200_ENOMEM;
    }
    e->arena_bytes = off;
    char* b = e->arena;
    e->x = (float*)(b + o_x); e->h = (float*)(b + o_h); e->qk = (float*)(b + o_qk); e->att = (float*)(b + o_att);
    e->y = (float*)(b + o_y); e->z = (float*)(b + o_z); e->sel_w = (float*)(b + o_sel_w); e->sel_e = (int*)(b + o_sel_e);
    e->slot_of = (int*)(b + o_slot_of); e->a_row = (int*)(b + o_a_row); e->a_scale = (float*)(b + o_a_scale);
    e->a_expert = (int*)(b + o_a_expert); e->n_slots = (int*)(b + o_n_slots); e->gu = (float*)(b + o_gu);
    e->mid = (float*)(b + o_mid); e->parts = (float*)(b + o_parts); e->sgu = (float*)(b + o_sgu);
    e->smid = (float*)(b + o_smid); e->hw = (float*)(b + o_hw);
    e->hb = b + o_hb; e->attb = b + o_attb; e->packb = b + o_packb; e->midb = b + o_midb; e->smidb = b + o_smidb;
    e->hwb = b + o_hwb;
    e->x0 = (float*)(b + o_x0); e->cat = (float*)(b + o_cat); e->proj = (float*)(b + o_proj); e->rec = (float*)(b + o_rec);
    e->outcat = (float*)(b + o_outcat); e->catb = b + o_catb; e->outcatb = b + o_outcatb;
    e->xs = (float*)(b + o_xs); e->qlat = (float*)(b + o_qlat); e->olat = (float*)(b + o_olat); e->floorb = (float*)(b + o_floor);
    e->unit = (float*)(b + o_unit); e->cqb = b + o_cqb;
    e->ymix = (float*)(b + o_ymix); e->h2 = (float*)(b + o_h2); e->h2b = b + o_h2b;
    e->split_ws = (float*)(b + o_split);
    e->split_arrived = (unsigned*)(b + o_arrived);
    const float unit_host[2] = {0.f, 1.f};
    if (cudaMemset(e->split_arrived, 0, arrived_bytes) != cudaSuccess ||
        cudaMemcpy(e->unit, unit_host, sizeof(unit_host), cudaMemcpyHostToDevice) != cudaSuccess) {
        (void)cudaGetLastError();
        cudaFree(e->arena);
        delete e;
        return LM_B200_ECUDA;
    }
    e->step_static = (int32_t*)(b + o_step);
    e->logits_static = (float*)(b + o_logits);
    *out = e;
    return LM_B200_OK;
}

int lm_b200_engine_destroy(lm_b200_engine* e) {
    if (!e) return LM_B200_OK;
    Guard g(e->device);
    for (auto& kv : e->graphs) cudaGraphExecDestroy(kv.second.exec);
    if (e->capture_stream) cudaStreamDestroy(e->capture_stream);
    if (e->arena) cudaFree(e->arena);
    delete e;
    return LM_B200_OK;
}

size_t lm_b200_engine_workspace_bytes(const lm_b200_engine* e) { return e ? e->arena_bytes : 0; }

}  // extern "C"

namespace {

// the final norm of the wanted rows of e->x and the logits
int head_rows(lm_b200_engine* e, const StepView& v, int n_want, float* logits_out, cudaStream_t st) {
    const int D = e->m.width;
    if (n_want > 0) {
        // the head is the largest single weight stream: from kHeadTensorRowsMin wanted rows on (a batch of decoding
        // sequences) the tensor-core kernel reads it once for all rows, where the row kernel reads it once per row
        const bool tc = e->m.precision == LM_B200_PRECISION_BF16 && n_want >= kHeadTensorRowsMin &&
                        dia::gemm_tcgen05_shape_ok(n_want, e->m.vocab, D) && (reinterpret_cast<uintptr_t>(logits_out) & 15) == 0;
        if (e->m.final_norm.kind == LM_B200_NORM_LAYER || e->m.final_norm.kind == LM_B200_NORM_RMS)
            LCK(lm::launch_layernorm_rows(e->x, v.want, e->m.final_norm.w, e->m.final_norm.b, e->m.eps,
                                          e->m.logit_scale != 0.f ? e->m.logit_scale : 1.f, e->hw, tc ? e->hwb : nullptr, n_want, D, st,
                                          e->m.final_norm.kind == LM_B200_NORM_RMS));
        else
            LCK(lm::launch_dyt_gather(e->x, v.want, N(e->m.final_norm), e->hw, tc ? e->hwb : nullptr, n_want, D, st));
        if (tc)
            LCK(dia::launch_gemm_tcgen05_bf16(e->hwb, 1, e->m.head, e->m.vocab, logits_out, n_want, e->m.vocab, D, kPlain, nullptr, st));
        else
            LCK(lm::launch_linear(e->hw, D, e->m.head, 0, logits_out, e->m.vocab, n_want, e->m.vocab, D, nullptr, st));
    }
    return LM_B200_OK;
}


// every layer of a stream-form model: the streams end up summed in e->x
int run_stream_layers(lm_b200_engine* e, const StepView& v, int M, int n_seq, float* layers_out, cudaStream_t st) {
    const int D = e->m.width, s = e->layers[0].streams, n = e->m.n_layer;
    const float eps = e->m.eps;
    const bool bf = e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin;
    void* hb = bf ? e->hb : nullptr;
    void* h2b = bf ? e->h2b : nullptr;
    LCK(lm::launch_streams_embed(e->m.embed, v.token, e->m.embed_scale != 0.f ? e->m.embed_scale : 1.f, e->xs, s, M, e->m.vocab, D, st,
                                 e->m.embed_norm, eps));
    const lm::StreamWrite none{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0};
    // A parallel record's feed-forward reads the streams the mixer read.  With one stream and one set of read weights both
    // norms share their statistics, and the step that produces the mixer's input writes the feed-forward's beside it.
    auto shares_read = [&](const lm_b200_layer& l) {
        return l.parallel && l.ff != LM_B200_FF_NONE && s == 1 && l.hc_in[0] == l.hc_in[1];
    };
    auto read_of = [&](const lm_b200_layer& l, lm::StreamExtra ex) {
        ex.rms = l.norm_mix_in.kind == LM_B200_NORM_RMS;
        if (shares_read(l)) { ex.norm_w2 = l.norm_ff_in.w; ex.h2 = e->h2; ex.h2_b = h2b; }
        return ex;
    };
    LCK(lm::launch_streams_step(e->xs, s, none, e->layers[0].hc_in[0], e->layers[0].norm_mix_in.w, eps, nullptr, e->h, hb, M, D, st,
                                read_of(e->layers[0], lm::StreamExtra{})));
    for (int i = 0; i < n; ++i) {
        const lm_b200_layer& l = e->layers[i];
        const bool par = l.parallel && l.ff != LM_B200_FF_NONE;
        int rc = stream_mixer(e, l, e->h, hb, v, M, n_seq, par ? e->ymix : e->y, st);
        if (rc) return rc;
        lm::StreamWrite wr{l.hc_mix[0], l.hc_out[0], e->y, nullptr, nullptr, nullptr, 0};
        lm::StreamExtra wx{};
        if (par) {
            if (!shares_read(l)) {
                lm::StreamExtra rx{};
                rx.rms = l.norm_ff_in.kind == LM_B200_NORM_RMS;
                LCK(lm::launch_streams_step(e->xs, s, none, l.hc_in[1], l.norm_ff_in.w, eps, nullptr, e->h2, h2b, M, D, st, rx));
            }
            rc = stream_ff(e, l, e->h2, h2b, M, &wr, &wx, st);
            if (rc) return rc;
            // one write for both sublayers: the streams mix once, the feed-forward's output goes in with its own write weights
            // and the mixer's beside it with the mixer's
            wr.out = l.hc_out[1];
            wx.y2 = e->ymix;
            wx.out2 = l.hc_out[0];
        } else if (l.ff != LM_B200_FF_NONE) {
            lm::StreamExtra rx{};
            rx.rms = l.norm_ff_in.kind == LM_B200_NORM_RMS;
            LCK(lm::launch_streams_step(e->xs, s, wr, l.hc_in[1], l.norm_ff_in.w, eps, nullptr, e->h, hb, M, D, st, rx));
            rc = stream_ff(e, l, e->h, hb, M, &wr, &wx, st);
            if (rc) return rc;
            wr.mix = l.hc_mix[1];
            wr.out = l.hc_out[1];
        }
        // this sublayer's write with the next layer's read, or with the closing sum of the streams
        if (i + 1 < n) {
            const lm_b200_layer& nx = e->layers[i + 1];
            LCK(lm::launch_streams_step(e->xs, s, wr, nx.hc_in[0], nx.norm_mix_in.w, eps, nullptr, e->h, hb, M, D, st, read_of(nx, wx)));
            if (layers_out)
                LCK(lm::launch_streams_step(e->xs, s, none, nullptr, nullptr, eps, nullptr, layers_out + (size_t)i * M * D, nullptr, M, D, st));
        } else {
            LCK(lm::launch_streams_step(e->xs, s, wr, nullptr, nullptr, eps, nullptr, e->x, nullptr, M, D, st, wx));
            if (layers_out && cudaMemcpyAsync(layers_out + (size_t)i * M * D, e->x, (size_t)M * D * 4, cudaMemcpyDeviceToDevice, st) !=
                                  cudaSuccess)
                return cuda_fail(cudaGetLastError());
        }
    }
    return LM_B200_OK;
}

// the launch sequence of one step
int run_step(lm_b200_engine* e, const int32_t* step, int M, int n_seq, int n_want, float* logits_out, float* layers_out,
             cudaStream_t st) {
    const StepView v = view(step, M, n_seq);
    const int D = e->m.width;
    if (e->stream_form) {
        const int rc = run_stream_layers(e, v, M, n_seq, layers_out, st);
        if (rc) return rc;
        return head_rows(e, v, n_want, logits_out, st);
    }
    LCK(lm::launch_embed(e->m.embed, v.token, e->x, M, e->m.vocab, D, st));
    bool keep_x0 = false;
    for (const lm_b200_layer& l : e->layers) keep_x0 = keep_x0 || (l.form == LM_B200_FORM_PARALLEL && l.w_pre);
    if (keep_x0 && cudaMemcpyAsync(e->x0, e->x, (size_t)M * D * 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return cuda_fail(cudaGetLastError());
    // Pure decoding (every scheduled sequence brings one row): the kernel that finishes a sublayer's residual add also
    // writes the next sublayer's input and moves its tail, so the norm + taps launches between sublayers fall away.
    const bool chain = M <= lm::kRowsKernelMax && n_seq == M;
    const lm::TapOut none{};
    bool h_ready = false;
    for (int i = 0; i < e->m.n_layer; ++i) {
        const lm_b200_layer& l = e->layers[i];
        if (l.form == LM_B200_FORM_PARALLEL) {
            const int prc = parallel_layer(e, l, v, M, n_seq, 0, nullptr, nullptr, st);
            if (prc) return prc;
            h_ready = false;
            if (layers_out && cudaMemcpyAsync(layers_out + (size_t)i * M * D, e->x, (size_t)M * D * 4, cudaMemcpyDeviceToDevice,
                                              st) != cudaSuccess)
                return cuda_fail(cudaGetLastError());
            continue;
        }
        const bool has_ff = l.ff == LM_B200_FF_ROUTED_EXPERTS, has_next = i + 1 < e->m.n_layer && e->layers[i + 1].form == LM_B200_FORM_SEQUENTIAL;
        int rc = LM_B200_OK;
        if (!h_ready) rc = norm_tapmix(e, l, 0, e->x, v, M, n_seq, e->h, st);
        if (rc) return rc;
        const void* hb = (e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin) ? e->hb : nullptr;
        const lm::TapOut after_mixer = !chain ? none : has_ff ? tap_out(e, l, 1, v) : has_next ? tap_out(e, e->layers[i + 1], 0, v) : none;
        rc = mixer(e, l, e->h, hb, v, M, e->y, e->x, after_mixer, st);
        if (rc) return rc;
        h_ready = after_mixer.h != nullptr;
        if (has_ff) {
            if (!h_ready) rc = norm_tapmix(e, l, 1, e->x, v, M, n_seq, e->h, st);
            if (rc) return rc;
            const lm::TapOut after_ff = (chain && has_next) ? tap_out(e, e->layers[i + 1], 0, v) : none;
            rc = feed_forward(e, l, e->h, hb, M, e->x, &l.norm_ff_out, after_ff, st);
            if (rc) return rc;
            h_ready = after_ff.h != nullptr;
        }
        if (layers_out) {
            if (cudaMemcpyAsync(layers_out + (size_t)i * M * D, e->x, (size_t)M * D * 4, cudaMemcpyDeviceToDevice, st) !=
                cudaSuccess)
                return cuda_fail(cudaGetLastError());
        }
    }
    return head_rows(e, v, n_want, logits_out, st);
}

// A step of a few rows is some forty short dependent launches: it is captured once per (rows, sequences, wanted) over
// the engine's fixed step and logits buffers and replayed as one graph launch; the step description is copied in and
// the logits out around it.
int run_step_graph(lm_b200_engine* e, const int32_t* step, int M, int n_seq, int n_want, float* logits_out, cudaStream_t st) {
    const size_t n_ints = 4 * (size_t)M + 3 * (size_t)n_seq + (size_t)n_want;
    if (cudaMemcpyAsync(e->step_static, step, n_ints * 4, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return cuda_fail(cudaGetLastError());
    const auto key = std::make_tuple(M, n_seq, n_want);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        if (!e->capture_stream && cudaStreamCreateWithFlags(&e->capture_stream, cudaStreamNonBlocking) != cudaSuccess)
            return cuda_fail(cudaGetLastError());
        cudaStream_t cs = e->capture_stream;
        if (cudaStreamBeginCapture(cs, cudaStreamCaptureModeRelaxed) != cudaSuccess) return cuda_fail(cudaGetLastError());
        const long long before = g_launches.load();
        const int rc = run_step(e, e->step_static, M, n_seq, n_want, e->logits_static, nullptr, cs);
        const long long launches = g_launches.load() - before;
        cudaGraph_t graph = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(cs, &graph);
        if (rc != LM_B200_OK || ce != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            return rc != LM_B200_OK ? rc : cuda_fail(ce != cudaSuccess ? ce : cudaErrorUnknown);
        }
        cudaGraphExec_t exec = nullptr;
        const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ie != cudaSuccess) return cuda_fail(ie);
        g_launches -= launches;                              // captured, not run: every replay counts them
        it = e->graphs.emplace(key, lm_b200_engine::StepGraph{exec, launches}).first;
    }
    if (cudaGraphLaunch(it->second.exec, st) != cudaSuccess) return cuda_fail(cudaGetLastError());
    g_launches += it->second.launches;
    if (n_want > 0 && cudaMemcpyAsync(logits_out, e->logits_static, (size_t)n_want * e->m.vocab * 4, cudaMemcpyDeviceToDevice,
                                      st) != cudaSuccess)
        return cuda_fail(cudaGetLastError());
    return LM_B200_OK;
}

}  // namespace

extern "C" {

int lm_b200_forward(lm_b200_engine* e, const int32_t* step, int M, int n_seq, int n_want, float* logits_out, float* layers_out,
                    void* stream) {
    if (!e || !step || M <= 0 || M > e->m.max_rows || n_seq <= 0 || n_seq > M || n_want < 0 || n_want > M ||
        (n_want > 0 && !logits_out))
        return LM_B200_EINVAL;
    Guard g(e->device);
    if (!g.ok) return LM_B200_ECUDA;
    if (e->m.step_graphs && M <= lm::kRowsKernelMax && !layers_out)
        return run_step_graph(e, step, M, n_seq, n_want, logits_out, S(stream));
    return run_step(e, step, M, n_seq, n_want, logits_out, layers_out, S(stream));
}

int lm_b200_op_norm_tapmix(lm_b200_engine* e, int layer, int sub, const float* x, const int32_t* step, int M, int n_seq,
                           float* out, void* stream) {
    if (!e || layer < 0 || layer >= e->m.n_layer || (sub != 0 && sub != 1) || !x || !step || !out || M <= 0 ||
        M > e->m.max_rows || n_seq <= 0)
        return LM_B200_EINVAL;
    Guard g(e->device);
    if (!g.ok) return LM_B200_ECUDA;
    if (e->layers[layer].form != LM_B200_FORM_SEQUENTIAL) return LM_B200_EUNSUPPORTED;
    return norm_tapmix(e, e->layers[layer], sub, x, view(step, M, n_seq), M, n_seq, out, S(stream));
}

int lm_b200_op_mixer(lm_b200_engine* e, int layer, const float* h, const int32_t* step, int M, int n_seq, float* y,
                     void* stream) {
    if (!e || layer < 0 || layer >= e->m.n_layer || !h || !step || !y || M <= 0 || M > e->m.max_rows || n_seq <= 0)
        return LM_B200_EINVAL;
    Guard g(e->device);
    if (!g.ok) return LM_B200_ECUDA;
    if (e->layers[layer].form == LM_B200_FORM_PARALLEL)
        return parallel_layer(e, e->layers[layer], view(step, M, n_seq), M, n_seq, 1, h, y, S(stream));
    if (e->layers[layer].form == LM_B200_FORM_STREAMS) {
        const void* hb = nullptr;
        if (e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin) {
            LCK(lm::launch_pack_rows_bf16(h, e->hb, M, e->m.width, nullptr, S(stream)));
            hb = e->hb;
        }
        return stream_mixer(e, e->layers[layer], h, hb, view(step, M, n_seq), M, n_seq, y, S(stream));
    }
    return mixer(e, e->layers[layer], h, nullptr, view(step, M, n_seq), M, y, nullptr, lm::TapOut{}, S(stream));
}

int lm_b200_op_attention(lm_b200_engine* e, int layer, float* qk, const int32_t* step, int M, int n_seq, float* out,
                         void* stream) {
    if (!e || layer < 0 || layer >= e->m.n_layer || !qk || !step || !out || M <= 0 || M > e->m.max_rows || n_seq <= 0)
        return LM_B200_EINVAL;
    Guard g(e->device);
    if (!g.ok) return LM_B200_ECUDA;
    const lm_b200_layer& l = e->layers[layer];
    if (l.form != LM_B200_FORM_SEQUENTIAL) return LM_B200_EUNSUPPORTED;
    const StepView v = view(step, M, n_seq);
    const int nq = l.heads * l.dim, nk = l.kv_heads * l.dim;
    const lm::PageMap pm{e->m.page_table, e->m.max_pages, e->m.page_size};
    LCK(lm::launch_qk_norm_cache(qk, nq, nk, l.q_norm, l.k_norm, e->m.eps, l.k_pages, l.v_pages, pm, l.kv_heads, l.dim, v.rm, M,
                                 S(stream)));
    const lm::AttnShape a{l.heads, l.kv_heads, l.dim, l.window, l.keep_first, l.scale, l.softcap, l.temp, l.slopes, l.sink};
    LCK(lm::launch_sink_attention(qk, nq + nk, l.k_pages, l.v_pages, pm, a, v.rm, out, nullptr, e->split_ws, e->split_arrived, M, S(stream)));
    return LM_B200_OK;
}

int lm_b200_op_mixer_kernels(lm_b200_engine* e, int layer, float* proj, const int32_t* step, int M, int n_seq, float* out,
                             void* stream) {
    if (!e || layer < 0 || layer >= e->m.n_layer || !proj || !step || !out || M <= 0 || M > e->m.max_rows || n_seq <= 0)
        return LM_B200_EINVAL;
    const lm_b200_layer& l = e->layers[layer];
    if (l.form != LM_B200_FORM_PARALLEL) return LM_B200_EUNSUPPORTED;
    Guard g(e->device);
    if (!g.ok) return LM_B200_ECUDA;
    const int rc = mixer_kernels(e, l, in_cols(l), proj, view(step, M, n_seq), M, n_seq, nullptr, S(stream));
    if (rc) return rc;
    const size_t w = (size_t)l.heads * l.vdim * 4;
    if (cudaMemcpy2DAsync(out, w, e->outcat, (size_t)l.k_out * 4, w, M, cudaMemcpyDeviceToDevice, S(stream)) != cudaSuccess)
        return cuda_fail(cudaGetLastError());
    return LM_B200_OK;
}

int lm_b200_op_ff(lm_b200_engine* e, int layer, const float* h, int M, float* y, void* stream) {
    if (!e || layer < 0 || layer >= e->m.n_layer || !h || !y || M <= 0 || M > e->m.max_rows) return LM_B200_EINVAL;
    const lm_b200_layer& l = e->layers[layer];
    if (l.form == LM_B200_FORM_PARALLEL) {
        if (l.ff != LM_B200_FF_DENSE) return LM_B200_EINVAL;
        Guard g(e->device);
        if (!g.ok) return LM_B200_ECUDA;
        return parallel_layer(e, l, StepView{}, M, 0, 2, h, y, S(stream));
    }
    if (l.form == LM_B200_FORM_STREAMS) {
        if (l.ff == LM_B200_FF_NONE) return LM_B200_EINVAL;
        Guard g(e->device);
        if (!g.ok) return LM_B200_ECUDA;
        const void* hb = nullptr;
        if (e->m.precision == LM_B200_PRECISION_BF16 && M >= kTensorRowsMin) {
            LCK(lm::launch_pack_rows_bf16(h, e->hb, M, e->m.width, nullptr, S(stream)));
            hb = e->hb;
        }
        lm::StreamWrite wr{};
        lm::StreamExtra wx{};
        const int rc = stream_ff(e, l, h, hb, M, &wr, &wx, S(stream));
        if (rc) return rc;
        // y = 0 * y + 1 * (the unit's output + the weighted expert outputs): one stream, mix {0}, out {1}
        if (cudaMemsetAsync(y, 0, (size_t)M * e->m.width * 4, S(stream)) != cudaSuccess) return cuda_fail(cudaGetLastError());
        wr.mix = e->unit;
        wr.out = e->unit + 1;
        LCK(lm::launch_streams_step(y, 1, wr, nullptr, nullptr, e->m.eps, nullptr, nullptr, nullptr, M, e->m.width, S(stream), wx));
        return LM_B200_OK;
    }
    if (l.ff != LM_B200_FF_ROUTED_EXPERTS) return LM_B200_EINVAL;
    Guard g(e->device);
    if (!g.ok) return LM_B200_ECUDA;
    return feed_forward(e, l, h, nullptr, M, y, nullptr, lm::TapOut{}, S(stream));                // no norm: the plain sum, written to y
}

int lm_b200_op_linear(const float* A, const void* W_bf16, float* Y, int M, int N, int K, void* stream) {
    if (!A || !W_bf16 || !Y || M <= 0 || N <= 0 || K <= 0) return LM_B200_EINVAL;
    LCK(lm::launch_linear(A, K, W_bf16, 0, Y, N, M, N, K, nullptr, S(stream)));
    return LM_B200_OK;
}

int lm_b200_op_linear_tc(const float* A, const void* W_bf16, float* Y, void* a_bf16, int M, int N, int K, void* stream) {
    if (!A || !W_bf16 || !Y || !a_bf16 || M <= 0 || N <= 0 || K <= 0) return LM_B200_EINVAL;
    if (!dia::gemm_tcgen05_shape_ok(M, N, K)) return LM_B200_EUNSUPPORTED;
    LCK(lm::launch_pack_rows_bf16(A, a_bf16, M, K, nullptr, S(stream)));
    LCK(dia::launch_gemm_tcgen05_bf16(a_bf16, 1, W_bf16, N, Y, M, N, K, kPlain, nullptr, S(stream)));
    return LM_B200_OK;
}

int lm_b200_argmax_rows(const float* logits, int M, int V, int32_t* out, void* stream) {
    if (!logits || !out || M <= 0 || V <= 0) return LM_B200_EINVAL;
    LCK(lm::launch_argmax_rows(logits, M, V, out, S(stream)));
    return LM_B200_OK;
}

}  // extern "C"

// lm_mixers.cu - kernels of the parallel layer form of the language-model path (sm_100a): layer norm, the attention whose
// scores are mixed across heads, the two recurrent mixers and the dense feed-forward's activation.
//
// Same step layout and the same rule as lm_kernels.cu: every kernel computes a row's result from that row and the
// sequence state it points at, in an order of operations that does not depend on what else is in the batch.  Positions,
// angles, norms, scores, softmax, gates, decays and the recurrent state are fp32.
//
//   layernorm_rows_kernel     (x - mean) / sqrt(var + eps) * w + b of (gathered) rows, fp32 and the bf16 GEMM operand
//   pair_rows_kernel          [x | x0] rows: the operand of the input mix in front of a repeated block
//   add_rows_kernel           x += y
//   talk_prep_kernel          q / k / v biases, per-head RMS norm of q and k, rotary positions on the leading channels
//                             (pairs 2i, 2i+1), k and v into the pages, sigmoid of the per-head output gate
//   talk_attention_kernel     softmax attention over the pages for ALL heads of a tile of rows at once: raw scores per
//                             head, mixed across heads by a [heads][heads] matrix, causal mask, online softmax with a
//                             value-less sink term, P.V per head, output gate.  A handful of rows (decoding) split their
//                             keys over CTAs and the last-arriving CTA merges the partial results.
//   delta_prep_kernel         short causal convolution + silu of q, k, v (previous inputs from the step or the sequence's
//                             tail), unit-vector q and k per head, beta, the per-channel decay and the output gate from
//                             their two-step projections
//   conv_tail_kernel          keeps the last taps-1 projected inputs of every scheduled sequence
//   gate_prep_kernel          silu(q), the bounded forget gate and biases of the gate-tied recurrence, in place
//   column_scan_kernel        the recurrence of both recurrent mixers, one value column of one head per 8 lanes:
//                             S <- a S;  [u = beta (v - S^T k)];  S <- S + w u;  o = S^T q, state carried per sequence
//   scalar_gate_scan_kernel   the same column layout for a recurrence with one decay and one write strength per token and
//                             head, and a normaliser carried as one more value column
//                             (or a fixed decay per head, write strength 1, no normaliser: retention)
//   head_norm_gate_kernel     per-head RMS norm of the read-out (x weight, x gate or its sigmoid / silu), fp32 in place and
//                             the bf16 operand
//   xielu_rows_kernel         the dense feed-forward's activation (xIELU or squared relu) on its slice of the stacked
//                             projections
// talk_attention_kernel also serves attention over cached latent rows (one key/value head whose value rows are the leading
// channels of its key rows) and takes a window; delta_prep_kernel and column_scan_kernel also serve the delta rule with ONE
// decay per head; layernorm_rows_kernel also computes the RMS norm.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "lm_device.cuh"
#include "lm_internal.h"

namespace lm {

// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                      const float* __restrict__ b, float eps, float out_scale, float* __restrict__ out,
                      __nv_bfloat16* __restrict__ out_b, int D, int rms) {
    __shared__ float red[32];
    pdl_release();
    pdl_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + (size_t)r * D;
    float s = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) s += xr[c];
    const float total = block_sum(s, red);
    const float mean = rms ? 0.f : total / (float)D;          // rms: x / sqrt(mean(x^2) + eps), no mean taken off
    float v = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float d = xr[c] - mean;
        v = fmaf(d, d, v);
    }
    const float inv = 1.0f / sqrtf(block_sum(v, red) / (float)D + eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float y = fmaf((xr[c] - mean) * inv, w[c], b ? b[c] : 0.f) * out_scale;
        out[(size_t)blockIdx.x * D + c] = y;
        if (out_b) out_b[(size_t)blockIdx.x * D + c] = __float2bfloat16_rn(y);
    }
}

__global__ void pair_rows_kernel(const float* __restrict__ x, const float* __restrict__ x0, float* __restrict__ cat,
                                 __nv_bfloat16* __restrict__ cat_b, int D) {
    pdl_release();
    pdl_wait();
    const size_t r = blockIdx.x;
    for (int c = threadIdx.x; c < 2 * D; c += blockDim.x) {
        const float v = c < D ? x[r * D + c] : x0[r * D + c - D];
        cat[r * 2 * D + c] = v;
        if (cat_b) cat_b[r * 2 * D + c] = __float2bfloat16_rn(v);
    }
}

__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
    pdl_release();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] += y[i];
}

__global__ void xielu_rows_kernel(const float* __restrict__ proj, int ld, int off, float ap, float an, float* __restrict__ out,
                                  int ldo, int out_off, __nv_bfloat16* __restrict__ out_b, int F, int relu2) {
    pdl_release();
    pdl_wait();
    const size_t r = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < F; c += gridDim.y * blockDim.x) {
        const float z = proj[r * ld + off + c];
        const float y = relu2 ? fmaxf(z, 0.f) * fmaxf(z, 0.f)
                              : z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
        if (out) out[r * ldo + out_off + c] = y;
        if (out_b) out_b[r * ldo + out_off + c] = __float2bfloat16_rn(y);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// One CTA per row, one warp per q / k head.  q <- rot(rms(q + bias) * qw) * scale in place (the score multiplier rides
// on q), k likewise without the multiplier into the key pages, v + bias into the value pages, gate <- sigmoid(gate).
__global__ void __launch_bounds__(256)
talk_prep_kernel(float* __restrict__ proj, int ld, const float* __restrict__ bias, int q_off, int k_off, int v_off, int gate_off,
                 int H, int G, int dim, int vdim, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                 float scale, const float* __restrict__ freq, int rot_dims, float* __restrict__ kcache,
                 float* __restrict__ vcache, const int* __restrict__ table, int max_pages, int page_size,
                 const int* __restrict__ row_slot, const int* __restrict__ row_pos) {
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    float* row = proj + (size_t)r * ld;
    const int pos = row_pos[r];
    const int page = table[(size_t)row_slot[r] * max_pages + pos / page_size], off = pos % page_size;
    for (int hh = warp; hh < H + G; hh += nwarp) {
        const bool isq = hh < H;
        const int base = isq ? q_off + hh * dim : k_off + (hh - H) * dim;
        float ss = 0.f;
        for (int c = lane; c < dim; c += 32) {
            const float v = row[base + c] + (bias ? bias[base + c] : 0.f);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
        const float* nw = isq ? qw : kw;
        const float mult = isq ? scale : 1.f;
        float* kdst = isq ? nullptr : kcache + (((size_t)page * G + (hh - H)) * page_size + off) * dim;
        for (int i = lane; 2 * i < dim; i += 32) {
            const int c0 = 2 * i, c1 = c0 + 1;
            float a = (row[base + c0] + (bias ? bias[base + c0] : 0.f)) * inv * nw[c0];
            float b = c1 < dim ? (row[base + c1] + (bias ? bias[base + c1] : 0.f)) * inv * nw[c1] : 0.f;
            if (c1 < rot_dims) {
                float sn, cs;
                sincosf((float)pos * freq[i], &sn, &cs);
                const float ra = a * cs - b * sn, rb = b * cs + a * sn;
                a = ra;
                b = rb;
            }
            a *= mult;
            b *= mult;
            if (isq) {
                row[base + c0] = a;
                if (c1 < dim) row[base + c1] = b;
            } else {
                kdst[c0] = a;
                if (c1 < dim) kdst[c1] = b;
            }
        }
    }
    for (int c = tid; c < G * vdim; c += blockDim.x) {
        const int g = c / vdim, d = c - g * vdim;
        vcache[(((size_t)page * G + g) * page_size + off) * vdim + d] = row[v_off + c] + (bias ? bias[v_off + c] : 0.f);
    }
    if (gate_off >= 0)
        for (int h = tid; h < H; h += blockDim.x) row[gate_off + h] = sigmoidf_(row[gate_off + h] + (bias ? bias[gate_off + h] : 0.f));
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention for all heads of a tile of TQ rows.  A (head, row) pair p = h * TQ + i owns one row of the score tiles and
// of the running statistics.  Per tile of 64 keys:
//   A  per key/value head g: the key tile is gathered from the pages into shared memory (asynchronous copies into one of
//      two buffers, issued a stage ahead); raw[p][j] = q_p . k_j for the pairs of the heads that read g (q carries the
//      score multiplier)
//   B  one warp per pair: mixed[p][j] = sum_g talk[h][g] raw[(g, i)][j], causal mask, online softmax (the running maximum
//      starts at the sink), weights to shared memory
//   C  per key/value head g: the value tile is gathered; out[p] += weights[p] . V for the pairs the warp owns (pair
//      w + 8 n of warp w: accumulators stay in registers across the whole key range)
// The rows of a tile may belong to several sequences: a maximal run of rows with one slot and consecutive positions is a
// segment, segments are walked one after the other and a row's statistics move only while its own segment is walked.
// With gridDim.y > 1 (TQ == 1, decoding) every CTA takes a share of the row's keys, writes {maximum, denominator,
// sums[vdim]} per head, and the CTA that arrives last merges the shares in their fixed order and adds the sink.
constexpr int kTalkTK = 64;

template <int VU, int NP, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
talk_attention_kernel(const float* __restrict__ proj, int ld, int q_off, int gate_off, const float* __restrict__ kcache,
                      const float* __restrict__ vcache, const int* __restrict__ table, int max_pages, int page_size, int H,
                      int G, int dim, int vdim, const float* __restrict__ talk, const float* __restrict__ sink,
                      const int* __restrict__ row_slot, const int* __restrict__ row_pos, float* __restrict__ out, int ldo,
                      __nv_bfloat16* __restrict__ out_b, int M, int TQ, float* __restrict__ part,
                      unsigned* __restrict__ arrived, int window) {
    extern __shared__ __align__(16) float sm[];
    __shared__ bool is_last;
    constexpr int TK = kTalkTK, NT = NW * 32;
    const int D4 = (dim + 3) >> 2, DQ = 4 * D4 + 4, SV = (vdim + 3) & ~3, kv_stride = max(DQ, SV);
    const int n_pairs = H * TQ, rep = H / G, tq_shift = 31 - __clz(TQ);       // TQ is a power of two
    float* Qs = sm;                                           // [n_pairs][DQ]
    float* KVs = Qs + (size_t)n_pairs * DQ;                   // [2][TK][kv_stride]: key and value tiles, double-buffered
    float* Rs = KVs + 2 * TK * kv_stride;                     // [n_pairs][TK] raw scores
    float* Ps = Rs + n_pairs * TK;                            // [n_pairs][TK] softmax weights
    float* m_s = Ps + n_pairs * TK;                           // [n_pairs] running maximum
    float* l_s = m_s + n_pairs;                               // [n_pairs] running denominator
    float* c_s = l_s + n_pairs;                               // [n_pairs] correction of this key tile
    float* Tm = c_s + n_pairs;                                // [H][H]
    int* s_slot = reinterpret_cast<int*>(Tm + H * H);         // [TQ]
    int* s_pos = s_slot + TQ;                                 // [TQ]

    pdl_release();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // later rows see more keys: their tiles start first
    const int r0 = (gridDim.x - 1 - blockIdx.x) * TQ, n_rows = min(TQ, M - r0), S = gridDim.y, sp = blockIdx.y;
    const bool vec_q = (dim % 4 == 0) && (ld % 4 == 0) && (q_off % 4 == 0), vec_k = dim % 4 == 0, vec_v = vdim % 4 == 0;
    // one key/value head whose value pages ARE its key pages (attention over a cached latent): the key tile of a stage
    // serves as its value tile, so a tile of keys is one gather and stays in its buffer through both phases
    // (a value row may also be the leading vdim channels of a wider key row)
    const bool shared_kv = kcache == vcache && G == 1 && vdim <= dim;

    if (tid < TQ) {
        s_slot[tid] = tid < n_rows ? row_slot[r0 + tid] : -1;
        s_pos[tid] = tid < n_rows ? row_pos[r0 + tid] : -1;
    }
    for (int i = tid; i < H * H; i += NT) Tm[i] = talk ? talk[i] : (i / H == i % H ? 1.f : 0.f);
    for (int idx = tid; idx < n_pairs * D4; idx += NT) {
        const int p = idx / D4, c = (idx - p * D4) * 4, h = p >> tq_shift, i = p & (TQ - 1);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n_rows) {
            const float* src = proj + (size_t)(r0 + i) * ld + q_off + (size_t)h * dim + c;
            if (vec_q) v = *reinterpret_cast<const float4*>(src);
            else {
                v.x = src[0];
                if (c + 1 < dim) v.y = src[1];
                if (c + 2 < dim) v.z = src[2];
                if (c + 3 < dim) v.w = src[3];
            }
        }
        *reinterpret_cast<float4*>(Qs + (size_t)p * DQ + c) = v;
    }
    for (int p = tid; p < n_pairs; p += NT) {
        m_s[p] = (S == 1 && sink) ? sink[p >> tq_shift] : -CUDART_INF_F;
        l_s[p] = 0.f;
    }
    // value columns of a lane: VW consecutive ones per group of 32 * VW columns (vector loads of the value tile)
    constexpr int VW = VU >= 4 ? 4 : VU;
    auto col_of = [&](int u) { return (u / VW) * 32 * VW + lane * VW + (u % VW); };
    float acc[NP][VU];
    int pg[NP];                                               // key/value head of owned pair n (-1: none)
#pragma unroll
    for (int n = 0; n < NP; ++n) {
        const int p = warp + NW * n;
        pg[n] = p < n_pairs ? (p >> tq_shift) / rep : -1;
#pragma unroll
        for (int u = 0; u < VU; ++u) acc[n][u] = 0.f;
    }
    __syncthreads();

    int seg_a = 0;
    while (seg_a < n_rows) {
        int seg_b = seg_a + 1;
        while (seg_b < n_rows && s_slot[seg_b] == s_slot[seg_a] && s_pos[seg_b] == s_pos[seg_b - 1] + 1) ++seg_b;
        const int* pages = table + (size_t)s_slot[seg_a] * max_pages;
        // with a window the segment's first row sees back to its position - window + 1, the later rows less far
        int k_begin = window > 0 ? max(0, s_pos[seg_a] - window + 1) : 0, k_end = s_pos[seg_b - 1] + 1;
        if (S > 1) {
            const int per = (k_end - k_begin + S - 1) / S;
            k_begin += sp * per;
            k_end = min(k_end, k_begin + per);
        }
        // A tile of 64 keys is 2 G stages: the key tiles of the G key/value heads (A), then their value tiles (C).  Stage
        // s lives in buffer s & 1; the gather of stage s + 1 is issued (asynchronous 16-byte copies, zero-filled beyond
        // the last key) before stage s is computed, so a stage's loads fly during the arithmetic of the one before.
        const int n_stage = k_begin < k_end ? ((k_end - k_begin + TK - 1) / TK) * 2 * G : 0;
        // a thread copies rows warp, warp + NW, ... of a tile and the 16-byte columns lane, lane + 32, ...; where a row
        // lives ((page * G) * page_size + offset in the page) is looked up once per tile, at its first stage
        int rowpg[TK / NW];
        auto gather = [&](int stg) {
            const int tile = stg / (2 * G), ph = stg - tile * 2 * G, j0 = k_begin + tile * TK, jn = min(TK, k_end - j0);
            if (ph == 0) {
#pragma unroll
                for (int i = 0; i < TK / NW; ++i) {
                    const int jj = warp + NW * i, j = j0 + jj;
                    rowpg[i] = jj < jn ? pages[j / page_size] * G * page_size + (j % page_size) : -1;
                }
            }
            const bool is_k = ph < G;
            if (shared_kv && !is_k) {
                asm volatile("cp.async.commit_group;" ::: "memory");
                return;
            }
            const int g = is_k ? ph : ph - G, width = is_k ? dim : vdim, W4 = is_k ? D4 : (SV >> 2);
            const float* cache = is_k ? kcache : vcache;
            const bool vec = is_k ? vec_k : vec_v;
            float* dstb = KVs + ((shared_kv ? tile : stg) & 1) * TK * kv_stride;
            for (int c4 = lane; c4 < W4; c4 += 32) {
                const int c = c4 * 4;
#pragma unroll
                for (int i = 0; i < TK / NW; ++i) {
                    float* dst = dstb + (warp + NW * i) * kv_stride + c;
                    const bool in = rowpg[i] >= 0;
                    const float* src = cache + (in ? ((size_t)rowpg[i] + (size_t)g * page_size) * width + c : 0);
                    if (vec) {
                        const unsigned d32 = (unsigned)__cvta_generic_to_shared(dst);
                        const int bytes = in ? 16 : 0;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d32), "l"(src), "r"(bytes) : "memory");
                    } else {
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (in) {
                            v.x = src[0];
                            if (c + 1 < width) v.y = src[1];
                            if (c + 2 < width) v.z = src[2];
                            if (c + 3 < width) v.w = src[3];
                        }
                        *reinterpret_cast<float4*>(dst) = v;
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (n_stage > 0) {
            __syncthreads();                                  // both buffers are free (the previous segment is done)
            gather(0);
        }
        for (int stg = 0; stg < n_stage; ++stg) {
            const int tile = stg / (2 * G), ph = stg - tile * 2 * G, j0 = k_begin + tile * TK, jn = min(TK, k_end - j0);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();                                  // stage stg has landed; stage stg - 1 is consumed
            if (stg + 1 < n_stage) gather(stg + 1);
            const float* KV = KVs + ((shared_kv ? tile : stg) & 1) * TK * kv_stride;
            if (ph < G) {
                // ---- A: raw scores of the heads that read key/value head g ----
                const int g = ph;
                const int np_g = rep * TQ;
                const float* Qg = Qs + (size_t)g * np_g * DQ;
                float* Rg = Rs + g * np_g * TK;
                if (np_g >= 32 && ((np_g + 3) / 4) * 2 > NW) {    // 4 pairs x 2 keys per thread
                    const float* k0p = KV + lane * kv_stride;
                    const float* k1p = KV + (lane + 32) * kv_stride;
                    for (int ch = warp; ch * 4 < np_g; ch += NW) {
                        const float* qp[4];
#pragma unroll
                        for (int a = 0; a < 4; ++a) qp[a] = Qg + (size_t)min(ch * 4 + a, np_g - 1) * DQ;
                        float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
                        for (int d4 = 0; d4 < D4; ++d4) {
                            const float4 k0 = *reinterpret_cast<const float4*>(k0p + 4 * d4);
                            const float4 k1 = *reinterpret_cast<const float4*>(k1p + 4 * d4);
#pragma unroll
                            for (int a = 0; a < 4; ++a) {
                                const float4 q = *reinterpret_cast<const float4*>(qp[a] + 4 * d4);
                                a0[a] = fmaf(q.x, k0.x, a0[a]); a0[a] = fmaf(q.y, k0.y, a0[a]);
                                a0[a] = fmaf(q.z, k0.z, a0[a]); a0[a] = fmaf(q.w, k0.w, a0[a]);
                                a1[a] = fmaf(q.x, k1.x, a1[a]); a1[a] = fmaf(q.y, k1.y, a1[a]);
                                a1[a] = fmaf(q.z, k1.z, a1[a]); a1[a] = fmaf(q.w, k1.w, a1[a]);
                            }
                        }
#pragma unroll
                        for (int a = 0; a < 4; ++a)
                            if (ch * 4 + a < np_g) {
                                Rg[(ch * 4 + a) * TK + lane] = a0[a];
                                Rg[(ch * 4 + a) * TK + lane + 32] = a1[a];
                            }
                    }
                } else if (np_g >= 32) {                      // fewer 4-pair chunks than half the warps: 4 pairs x 1 key
                    for (int it = warp; it * 2 < np_g; it += NW) {    // items: (chunk of 4 pairs, half of the keys)
                        const int ch = it >> 1, jj = lane + 32 * (it & 1);
                        const float* kp = KV + jj * kv_stride;
                        const float* qp[4];
#pragma unroll
                        for (int a = 0; a < 4; ++a) qp[a] = Qg + (size_t)min(ch * 4 + a, np_g - 1) * DQ;
                        float a0[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
                        for (int d4 = 0; d4 < D4; ++d4) {
                            const float4 k0 = *reinterpret_cast<const float4*>(kp + 4 * d4);
#pragma unroll
                            for (int a = 0; a < 4; ++a) {
                                const float4 q = *reinterpret_cast<const float4*>(qp[a] + 4 * d4);
                                a0[a] = fmaf(q.x, k0.x, a0[a]); a0[a] = fmaf(q.y, k0.y, a0[a]);
                                a0[a] = fmaf(q.z, k0.z, a0[a]); a0[a] = fmaf(q.w, k0.w, a0[a]);
                            }
                        }
#pragma unroll
                        for (int a = 0; a < 4; ++a)
                            if (ch * 4 + a < np_g) Rg[(ch * 4 + a) * TK + jj] = a0[a];
                    }
                } else {                                      // few pairs (decoding): 1 pair x 1 key per thread
                    for (int it = warp; it < 2 * np_g; it += NW) {
                        const int lp = it >> 1, jj = lane + 32 * (it & 1);
                        const float* qp = Qg + (size_t)lp * DQ;
                        const float* kp = KV + jj * kv_stride;
                        float a = 0.f;
                        if (jj < jn) {
                            for (int d4 = 0; d4 < D4; ++d4) {
                                const float4 q = *reinterpret_cast<const float4*>(qp + 4 * d4);
                                const float4 k = *reinterpret_cast<const float4*>(kp + 4 * d4);
                                a = fmaf(q.x, k.x, a); a = fmaf(q.y, k.y, a); a = fmaf(q.z, k.z, a); a = fmaf(q.w, k.w, a);
                            }
                        }
                        Rg[lp * TK + jj] = a;
                    }
                }
                if (ph < G - 1) continue;
                __syncthreads();                              // the raw scores of all heads are there
                // ---- B: mix across heads, mask, online softmax ----
                for (int p = warp; p < n_pairs; p += NW) {
                    const int h = p >> tq_shift, i = p & (TQ - 1);
                    const bool live = i >= seg_a && i < seg_b;
                    const int qi = s_pos[i];
                    float s[2];
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const int jj = lane + 32 * t;
                        const bool ok = live && jj < jn && j0 + jj <= qi && (window <= 0 || qi - (j0 + jj) < window);
                        float v = -CUDART_INF_F;
                        if (ok) {
                            if (talk) {
                                v = 0.f;
                                for (int g2 = 0; g2 < H; ++g2) v = fmaf(Tm[h * H + g2], Rs[(g2 * TQ + i) * TK + jj], v);
                            } else {
                                v = Rs[p * TK + jj];
                            }
                        }
                        s[t] = v;
                    }
                    const float m_old = m_s[p];
                    const float m_new = fmaxf(m_old, warp_max(fmaxf(s[0], s[1])));
                    float corr = 1.f, p0 = 0.f, p1 = 0.f;
                    if (m_new != -CUDART_INF_F) {
                        corr = expf(m_old - m_new);           // exp(-inf) = 0 on the first live tile without a sink
                        p0 = expf(s[0] - m_new);
                        p1 = expf(s[1] - m_new);
                    }
                    const float psum = warp_sum(p0 + p1);
                    Ps[p * TK + lane] = p0;
                    Ps[p * TK + lane + 32] = p1;
                    if (lane == 0) {
                        l_s[p] = l_s[p] * corr + psum;
                        m_s[p] = m_new;
                        c_s[p] = corr;
                    }
                }
                continue;                                     // the next stage's barrier publishes the weights
            }
            // ---- C: weighted values of key/value head g ----
            const int g = ph - G;
            const int jn4 = (jn + 3) & ~3;
#pragma unroll
            for (int n = 0; n < NP; ++n)
                if (pg[n] == g) {
                    const float c = c_s[warp + NW * n];
#pragma unroll
                    for (int u = 0; u < VU; ++u) acc[n][u] *= c;
                }
            // the pairs of one key/value head are neighbours in a warp's list: two at a time share the loaded values
#pragma unroll
            for (int n0 = 0; n0 < NP; n0 += 2) {
                const bool own0 = pg[n0] == g, own1 = n0 + 1 < NP && pg[n0 + 1 < NP ? n0 + 1 : n0] == g;
                if (!own0 && !own1) continue;
                const float* P0 = Ps + (warp + NW * n0) * TK;
                const float* P1 = Ps + (warp + NW * (n0 + 1 < NP ? n0 + 1 : n0)) * TK;
                for (int j = 0; j < jn4; j += 4) {
                    float v[4][VU];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
#pragma unroll
                        for (int u = 0; u < VU; u += VW) {
                            const int col = col_of(u);
                            const float* src = KV + (j + jj) * kv_stride + col;
                            if (VW == 4) {
                                const float4 t = col < SV ? *reinterpret_cast<const float4*>(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                                v[jj][u] = t.x; v[jj][u + 1] = t.y; v[jj][u + 2] = t.z; v[jj][u + 3] = t.w;
                            } else if (VW == 2) {
                                const float2 t = col < SV ? *reinterpret_cast<const float2*>(src) : make_float2(0.f, 0.f);
                                v[jj][u] = t.x; v[jj][u + 1] = t.y;
                            } else {
                                v[jj][u] = col < SV ? *src : 0.f;
                            }
                        }
                    if (own0) {
                        const float4 pj = *reinterpret_cast<const float4*>(P0 + j);
#pragma unroll
                        for (int u = 0; u < VU; ++u) {
                            acc[n0][u] = fmaf(pj.x, v[0][u], acc[n0][u]);
                            acc[n0][u] = fmaf(pj.y, v[1][u], acc[n0][u]);
                            acc[n0][u] = fmaf(pj.z, v[2][u], acc[n0][u]);
                            acc[n0][u] = fmaf(pj.w, v[3][u], acc[n0][u]);
                        }
                    }
                    if (own1) {
                        const float4 pj = *reinterpret_cast<const float4*>(P1 + j);
#pragma unroll
                        for (int u = 0; u < VU; ++u) {
                            float& dst = acc[n0 + 1 < NP ? n0 + 1 : n0][u];
                            dst = fmaf(pj.x, v[0][u], dst);
                            dst = fmaf(pj.y, v[1][u], dst);
                            dst = fmaf(pj.z, v[2][u], dst);
                            dst = fmaf(pj.w, v[3][u], dst);
                        }
                    }
                }
            }
        }
        seg_a = seg_b;
    }
    __syncthreads();

    if (S == 1) {                                             // the sink's own term, normalise, gate, store
#pragma unroll
        for (int n = 0; n < NP; ++n) {
            if (pg[n] < 0) continue;
            const int p = warp + NW * n, h = p >> tq_shift, i = p & (TQ - 1);
            if (i >= n_rows) continue;
            float l = l_s[p];
            if (sink) l += expf(sink[h] - m_s[p]);
            float f = l > 0.f ? 1.0f / l : 0.f;
            if (gate_off >= 0) f *= proj[(size_t)(r0 + i) * ld + gate_off + h];
            const size_t base = (size_t)(r0 + i) * ldo + (size_t)h * vdim;
#pragma unroll
            for (int u = 0; u < VU; ++u) {
                const int col = col_of(u);
                if (col < vdim) {
                    const float o = acc[n][u] * f;
                    out[base + col] = o;
                    if (out_b) out_b[base + col] = __float2bfloat16_rn(o);
                }
            }
        }
        return;
    }
    // ---- shares of a row's keys: part[((row * H + h) * S + share)] = {maximum, denominator, sums[vdim]} ----
    const size_t stride = (size_t)vdim + 2;
#pragma unroll
    for (int n = 0; n < NP; ++n) {
        if (pg[n] < 0) continue;
        const int p = warp + NW * n;                  // TQ == 1: the pair is the head
        float* dst = part + (((size_t)r0 * H + p) * S + sp) * stride;
        if (lane == 0) { dst[0] = m_s[p]; dst[1] = l_s[p]; }
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            const int col = col_of(u);
            if (col < vdim) dst[2 + col] = acc[n][u];
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned seen = atomicAdd(arrived + r0, 1u);
        is_last = seen == (unsigned)S - 1u;
        if (is_last) arrived[r0] = 0u;                        // back to zero for the next step
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int h = warp; h < H; h += NW) {
        const float* src = part + ((size_t)r0 * H + h) * S * stride;
        const float ms = lane < S ? __ldcg(src + lane * stride) : -CUDART_INF_F;
        const float ls = lane < S ? __ldcg(src + lane * stride + 1) : 0.f;
        const float sk = sink ? sink[h] : -CUDART_INF_F;
        const float m = fmaxf(sk, warp_max(ms));
        const float w = ms == -CUDART_INF_F ? 0.f : expf(ms - m);
        float l = sink ? expf(sk - m) : 0.f;
        for (int t = 0; t < S; ++t) l += __shfl_sync(0xffffffffu, ls * w, t);
        float f = l > 0.f ? 1.0f / l : 0.f;
        if (gate_off >= 0) f *= proj[(size_t)r0 * ld + gate_off + h];
        for (int c0 = 0; c0 < vdim; c0 += 32) {
            const int col = c0 + lane;
            float o = 0.f;
            for (int t = 0; t < S; ++t) {
                const float wt = __shfl_sync(0xffffffffu, w, t);
                if (col < vdim) o = fmaf(__ldcg(src + t * stride + 2 + col), wt, o);
            }
            if (col < vdim) {
                o *= f;
                out[(size_t)r0 * ldo + (size_t)h * vdim + col] = o;
                if (out_b) out_b[(size_t)r0 * ldo + (size_t)h * vdim + col] = __float2bfloat16_rn(o);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// One CTA per row.  Channels c of [q | k | v] (C = 2 G dim + H vdim, the first columns of the stacked projections):
//   conv_c = silu(sum_o cw[c][taps-1-o] * u_c(pos - o)),  u from the step's earlier rows or the sequence's tail, zero
//   before position 0;  q, k heads -> unit vectors (q also x dim^-1/2);  beta = sigmoid;  decay[h][d] =
//   exp(-exp(a_log[h]) softplus(z[h d] + dt_bias[h d]));  gate[h][c] = sigmoid(y[h c]), where z and y - the second steps
//   of the two-step decay and gate projections, fp32 products - already stand in the row's decay and gate columns.
// rec row: q (G dim) | k (G dim) | v (H vdim) | decay (H dim) | gate (H vdim) | beta (H)
__global__ void __launch_bounds__(256)
delta_prep_kernel(const float* __restrict__ proj, int ld, int beta_off, int H, int G, int dim, int vdim, int taps,
                  const float* __restrict__ cw, const float* __restrict__ tail, const float* __restrict__ a_log,
                  const float* __restrict__ dt_bias, float unit_eps, const int* __restrict__ row_slot,
                  const int* __restrict__ row_pos, const int* __restrict__ row_start, float* __restrict__ rec, int ldr,
                  int head_decay_off) {
    extern __shared__ float cbuf[];                           // [C] convolved + silu
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const int C = 2 * G * dim + H * vdim, T1 = taps - 1;
    const int slot = row_slot[r], pos = row_pos[r], start = row_start[r];
    const float* row = proj + (size_t)r * ld;
    float* dst = rec + (size_t)r * ldr;
    for (int c = tid; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int o = 0; o < taps; ++o) {
            const int p = pos - o;
            if (p < 0) break;
            const float u = p >= start ? proj[(size_t)(r - o) * ld + c]
                                       : tail[((size_t)slot * T1 + (p - (start - T1))) * C + c];
            acc = fmaf(cw[(size_t)c * taps + taps - 1 - o], u, acc);
        }
        cbuf[c] = siluf_(acc);
    }
    __syncthreads();
    const float qmul = 1.0f / sqrtf((float)dim);
    for (int hh = warp; hh < 2 * G; hh += nwarp) {            // q heads, then k heads
        const float* src = cbuf + hh * dim;
        float ss = 0.f;
        for (int c = lane; c < dim; c += 32) ss = fmaf(src[c], src[c], ss);
        ss = warp_sum(ss);
        const float inv = (hh < G ? qmul : 1.f) / sqrtf(ss + unit_eps);
        for (int c = lane; c < dim; c += 32) dst[hh * dim + c] = src[c] * inv;
    }
    if (head_decay_off >= 0) {
        // one decay per head, its pre-activation a column of the stacked projections; the output gate stays where it is.
        // rec row: q (G dim) | k (G dim) | v (H vdim) | decay (H) | beta (H)
        const int v0 = 2 * G * dim, d0 = v0 + H * vdim, b0 = d0 + H;
        for (int c = tid; c < H * vdim; c += blockDim.x) dst[v0 + c] = cbuf[v0 + c];
        for (int h = tid; h < H; h += blockDim.x) {
            dst[d0 + h] = expf(-expf(a_log[h]) * softplusf_(row[head_decay_off + h] + dt_bias[h]));
            dst[b0 + h] = sigmoidf_(row[beta_off + h]);
        }
        return;
    }
    const int v0 = 2 * G * dim, d0 = v0 + H * vdim, g0 = d0 + H * dim, b0 = g0 + H * vdim;
    for (int c = tid; c < H * vdim; c += blockDim.x) {
        dst[v0 + c] = cbuf[v0 + c];
        dst[g0 + c] = sigmoidf_(dst[g0 + c]);                  // the second step of the gate projection is already there
    }
    for (int c = tid; c < H * dim; c += blockDim.x)            // ... and that of the decay projection
        dst[d0 + c] = expf(-expf(a_log[c / dim]) * softplusf_(dst[d0 + c] + dt_bias[c]));
    for (int h = tid; h < H; h += blockDim.x) dst[b0 + h] = sigmoidf_(row[beta_off + h]);
}

// tail[slot][i][c] <- projected input at position (start + count) - (taps-1) + i of every scheduled sequence: from this
// step's rows when that position is in the step, else the old tail shifted by `count`
__global__ void conv_tail_kernel(const float* __restrict__ proj, int ld, int C, int taps, float* __restrict__ tail,
                                 const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                                 const int* __restrict__ seq_count) {
    pdl_release();
    pdl_wait();
    const int s = blockIdx.x, T1 = taps - 1;
    const int slot = seq_slot[s], row0 = seq_row0[s], n = seq_count[s];
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float keep[kMaxTaps];
        float* t = tail + (size_t)slot * T1 * C + c;
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) {
            if (i >= T1) break;
            const int q = n - T1 + i;
            keep[i] = q >= 0 ? proj[(size_t)(row0 + q) * ld + c] : t[(size_t)(i + n) * C];
        }
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) {
            if (i >= T1) break;
            t[(size_t)i * C] = keep[i];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// q <- silu(q + bias), f <- lower + (1 - lower) sigmoid(f + bias), v <- v + bias in place on the stacked projections of
// a gate-tied recurrence (one CTA per row): what its scan reads as q, decay and value
__global__ void gate_prep_kernel(float* __restrict__ proj, int ld, int q_off, int f_off, int v_off, const float* __restrict__ bias,
                                 const float* __restrict__ lower, int n_qf, int n_v) {
    pdl_release();
    pdl_wait();
    float* row = proj + (size_t)blockIdx.x * ld;
    for (int c = threadIdx.x; c < n_qf; c += blockDim.x) {
        row[q_off + c] = siluf_(row[q_off + c] + (bias ? bias[q_off + c] : 0.f));
        const float lo = lower ? lower[c] : 0.f;
        row[f_off + c] = fmaf(1.0f - lo, sigmoidf_(row[f_off + c] + (bias ? bias[f_off + c] : 0.f)), lo);
    }
    if (bias)
        for (int c = threadIdx.x; c < n_v; c += blockDim.x) row[v_off + c] += bias[v_off + c];
}

// The recurrence.  Per head a state S [dim][vdim]; every value column c of S evolves on its own:
//   S[:, c] <- a_t * S[:, c];   DELTA: u = beta_t (v_t[c] - S[:, c] . k_t), S[:, c] += k_t u;   else: S[:, c] += (1 - a_t) v_t[c]
//   o_t[c] = S[:, c] . q_t
// A column lives in the registers of 8 lanes (lane part holds rows part, part + 8, ...; its dot products are summed in
// four interleaved partial sums, then across the 8 lanes); a CTA of 4 warps carries 16 columns of one head of one
// scheduled sequence through the sequence's rows in order, 16 tokens staged in shared memory at a time while the next 16
// are on their way into registers.  The state is read when the sequence's first row is not position 0, and written
// back at the end: state[slot][h][c][dim].
constexpr int kScanThreads = 128, kScanCols = 16, kScanTT = 16;

template <int RP, bool DELTA>
__global__ void __launch_bounds__(kScanThreads)
column_scan_kernel(const float* __restrict__ in, int ld, int q_off, int k_off, int a_off, int v_off, int beta_off, int H, int G,
                   int dim, int vdim, float* __restrict__ state, const int* __restrict__ seq_slot,
                   const int* __restrict__ seq_row0, const int* __restrict__ seq_count, const int* __restrict__ row_pos,
                   float* __restrict__ o, int ldo, int head_decay) {
    extern __shared__ float sh[];
    constexpr int DS = 8 * RP;                                // staged row length (channels beyond dim hold zeros)
    float* sq = sh;                                           // [TT][DS]
    float* sa = sq + kScanTT * DS;                            // [TT][DS]
    float* sk = sa + kScanTT * DS;                            // [TT][DS] (DELTA)
    float* sv = sk + (DELTA ? kScanTT * DS : 0);              // [TT][16]
    float* sb = sv + kScanTT * kScanCols;                     // [TT] (DELTA)
    pdl_release();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kScanCols;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, part = lane & 7, cl = warp * 4 + (lane >> 3);
    const int col = col0 + cl, g = h / (H / G);
    const int slot = seq_slot[s], row0 = seq_row0[s], n = seq_count[s], start = row_pos[row0];
    const bool col_ok = col < vdim;
    float* st = state + (((size_t)slot * H + h) * vdim + (col_ok ? col : 0)) * dim;
    float S[RP];
#pragma unroll
    for (int r = 0; r < RP; ++r) {
        const int d = part + 8 * r;
        S[r] = (start > 0 && col_ok && d < dim) ? st[d] : 0.f;
    }
    // Staging: a chunk of 16 tokens is 16 * DS = 128 * RP elements per input; thread tid owns elements tid + 128 i, the
    // same (token in chunk, channel) for every chunk.
    int src[RP];                                              // (token in chunk) * ld + channel, -1: a channel beyond dim
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int idx = tid + kScanThreads * i, t = idx / DS, d = idx - t * DS;
        src[i] = d < dim ? t * ld + d : -1;
    }
    const int qh = DELTA ? g : h;
    float rq[RP], ra[RP], rk[DELTA ? RP : 1], rv[2], rb = 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(kScanTT, n - t0);
        const float* base = in + (size_t)(row0 + t0) * ld;
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            const bool ok = src[i] >= 0 && (tid + kScanThreads * i) / DS < nt;
            rq[i] = ok ? base[src[i] + q_off + qh * dim] : 0.f;
            // head_decay: column a_off + h of the row holds the one decay of all of the head's key channels
            ra[i] = !ok ? 0.f : head_decay ? base[((tid + kScanThreads * i) / DS) * ld + a_off + h] : base[src[i] + a_off + h * dim];
            if (DELTA) rk[i] = ok ? base[src[i] + k_off + g * dim] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + kScanThreads * i, t = idx / kScanCols, c = idx - t * kScanCols;
            rv[i] = (t < nt && col0 + c < vdim) ? base[(size_t)t * ld + v_off + h * vdim + col0 + c] : 0.f;
        }
        if (DELTA && tid < nt) rb = base[(size_t)tid * ld + beta_off + h];
    };
    fetch(0);
    for (int t0 = 0; t0 < n; t0 += kScanTT) {
        const int nt = min(kScanTT, n - t0);
        __syncthreads();                                      // the previous chunk is consumed
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            const int idx = tid + kScanThreads * i;
            sq[idx] = rq[i];
            sa[idx] = ra[i];
            if (DELTA) sk[idx] = rk[i];
        }
        sv[tid] = rv[0];
        sv[tid + kScanThreads] = rv[1];
        if (DELTA && tid < kScanTT) sb[tid] = rb;
        __syncthreads();
        if (t0 + kScanTT < n) fetch(t0 + kScanTT);            // in flight during the recurrence below
#pragma unroll 4
        for (int t = 0; t < nt; ++t) {
            const float* q = sq + t * DS + part;
            const float* a = sa + t * DS + part;
            const float v = sv[t * kScanCols + cl];
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
            if (DELTA) {
                const float* k = sk + t * DS + part;
                float e0 = 0.f, e1 = 0.f, e2 = 0.f, e3 = 0.f;
#pragma unroll
                for (int r = 0; r < RP; r += 4) {
                    S[r] *= a[8 * r];
                    S[r + 1] *= a[8 * r + 8];
                    S[r + 2] *= a[8 * r + 16];
                    S[r + 3] *= a[8 * r + 24];
                    e0 = fmaf(S[r], k[8 * r], e0);
                    e1 = fmaf(S[r + 1], k[8 * r + 8], e1);
                    e2 = fmaf(S[r + 2], k[8 * r + 16], e2);
                    e3 = fmaf(S[r + 3], k[8 * r + 24], e3);
                }
                float dk = (e0 + e1) + (e2 + e3);
                dk += __shfl_xor_sync(0xffffffffu, dk, 1);
                dk += __shfl_xor_sync(0xffffffffu, dk, 2);
                dk += __shfl_xor_sync(0xffffffffu, dk, 4);
                const float u = sb[t] * (v - dk);
#pragma unroll
                for (int r = 0; r < RP; r += 4) {
                    S[r] = fmaf(k[8 * r], u, S[r]);
                    S[r + 1] = fmaf(k[8 * r + 8], u, S[r + 1]);
                    S[r + 2] = fmaf(k[8 * r + 16], u, S[r + 2]);
                    S[r + 3] = fmaf(k[8 * r + 24], u, S[r + 3]);
                    d0 = fmaf(S[r], q[8 * r], d0);
                    d1 = fmaf(S[r + 1], q[8 * r + 8], d1);
                    d2 = fmaf(S[r + 2], q[8 * r + 16], d2);
                    d3 = fmaf(S[r + 3], q[8 * r + 24], d3);
                }
            } else {
#pragma unroll
                for (int r = 0; r < RP; r += 4) {
                    const float a0 = a[8 * r], a1 = a[8 * r + 8], a2 = a[8 * r + 16], a3 = a[8 * r + 24];
                    S[r] = fmaf(a0, S[r], (1.0f - a0) * v);
                    S[r + 1] = fmaf(a1, S[r + 1], (1.0f - a1) * v);
                    S[r + 2] = fmaf(a2, S[r + 2], (1.0f - a2) * v);
                    S[r + 3] = fmaf(a3, S[r + 3], (1.0f - a3) * v);
                    d0 = fmaf(S[r], q[8 * r], d0);
                    d1 = fmaf(S[r + 1], q[8 * r + 8], d1);
                    d2 = fmaf(S[r + 2], q[8 * r + 16], d2);
                    d3 = fmaf(S[r + 3], q[8 * r + 24], d3);
                }
            }
            float dot = (d0 + d1) + (d2 + d3);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            if (part == 0 && col_ok) o[(size_t)(row0 + t0 + t) * ldo + h * vdim + col] = dot;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < RP; ++r) {
            const int d = part + 8 * r;
            if (d < dim) st[d] = S[r];
        }
    }
}

// The same column layout for a recurrence with scalar gates per (token, head):  S[:, c] <- a_t S[:, c] + (b_t k_t) v_t[c],
// o_t[c] = S[:, c] . q_t.  Column vdim of every head is the normaliser: its value is the constant 1, so it carries
// n <- a n + b k and reads out n . q.  State and read-out have vdim + 1 columns per head: state[slot][h][c][dim].
template <int RP>
__global__ void __launch_bounds__(kScanThreads)
scalar_gate_scan_kernel(const float* __restrict__ in, int ld, int q_off, int k_off, int a_off, int v_off, int b_off, int H, int dim,
                        int vdim, float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                        const int* __restrict__ seq_count, const int* __restrict__ row_pos, float* __restrict__ o, int ldo,
                        const float* __restrict__ fixed_decay, int normaliser) {
    extern __shared__ float sh[];
    constexpr int DS = 8 * RP;
    float* sq = sh;                                           // [TT][DS]
    float* sk = sq + kScanTT * DS;                            // [TT][DS]
    float* sv = sk + kScanTT * DS;                            // [TT][16]
    float* sa = sv + kScanTT * kScanCols;                     // [TT]
    float* sb = sa + kScanTT;                                 // [TT]
    pdl_release();
    pdl_wait();
    // fixed_decay: a = fixed_decay[h] and b = 1 for every token (no gate columns are read); normaliser 0: vdim columns
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kScanCols, vcols = vdim + (normaliser ? 1 : 0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, part = lane & 7, cl = warp * 4 + (lane >> 3);
    const int col = col0 + cl;
    const int slot = seq_slot[s], row0 = seq_row0[s], n = seq_count[s], start = row_pos[row0];
    const bool col_ok = col < vcols;
    const float a_fix = fixed_decay ? fixed_decay[h] : 0.f;
    float* st = state + (((size_t)slot * H + h) * vcols + (col_ok ? col : 0)) * dim;
    float S[RP];
#pragma unroll
    for (int r = 0; r < RP; ++r) {
        const int d = part + 8 * r;
        S[r] = (start > 0 && col_ok && d < dim) ? st[d] : 0.f;
    }
    int src[RP];
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int idx = tid + kScanThreads * i, t = idx / DS, d = idx - t * DS;
        src[i] = d < dim ? t * ld + d : -1;
    }
    float rq[RP], rk[RP], rv[2], ra = 0.f, rb = 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(kScanTT, n - t0);
        const float* base = in + (size_t)(row0 + t0) * ld;
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            const bool ok = src[i] >= 0 && (tid + kScanThreads * i) / DS < nt;
            rq[i] = ok ? base[src[i] + q_off + h * dim] : 0.f;
            rk[i] = ok ? base[src[i] + k_off + h * dim] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + kScanThreads * i, t = idx / kScanCols, c = col0 + (idx - t * kScanCols);
            rv[i] = t < nt ? (c < vdim ? base[(size_t)t * ld + v_off + h * vdim + c] : ((c == vdim && normaliser) ? 1.f : 0.f)) : 0.f;
        }
        if (tid < nt) {
            ra = fixed_decay ? a_fix : base[(size_t)tid * ld + a_off + h];
            rb = fixed_decay ? 1.f : base[(size_t)tid * ld + b_off + h];
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < n; t0 += kScanTT) {
        const int nt = min(kScanTT, n - t0);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            const int idx = tid + kScanThreads * i;
            sq[idx] = rq[i];
            sk[idx] = rk[i];
        }
        sv[tid] = rv[0];
        sv[tid + kScanThreads] = rv[1];
        if (tid < kScanTT) { sa[tid] = ra; sb[tid] = rb; }
        __syncthreads();
        if (t0 + kScanTT < n) fetch(t0 + kScanTT);
#pragma unroll 4
        for (int t = 0; t < nt; ++t) {
            const float* q = sq + t * DS + part;
            const float* k = sk + t * DS + part;
            const float a = sa[t], u = sb[t] * sv[t * kScanCols + cl];
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int r = 0; r < RP; r += 4) {
                S[r] = fmaf(a, S[r], k[8 * r] * u);
                S[r + 1] = fmaf(a, S[r + 1], k[8 * r + 8] * u);
                S[r + 2] = fmaf(a, S[r + 2], k[8 * r + 16] * u);
                S[r + 3] = fmaf(a, S[r + 3], k[8 * r + 24] * u);
                d0 = fmaf(S[r], q[8 * r], d0);
                d1 = fmaf(S[r + 1], q[8 * r + 8], d1);
                d2 = fmaf(S[r + 2], q[8 * r + 16], d2);
                d3 = fmaf(S[r + 3], q[8 * r + 24], d3);
            }
            float dot = (d0 + d1) + (d2 + d3);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            if (part == 0 && col_ok) o[(size_t)(row0 + t0 + t) * ldo + h * vcols + col] = dot;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < RP; ++r) {
            const int d = part + 8 * r;
            if (d < dim) st[d] = S[r];
        }
    }
}

// o[r][h] <- o[r][h] / sqrt(mean(o[r][h]^2) + eps) * w [* gate[r][h]] in place (one warp per row and head), and its bf16 copy
// gate_act: 0 the gate columns are used as they are (already activated), 1 sigmoid, 2 silu of them; w may be absent
__global__ void head_norm_gate_kernel(float* __restrict__ o, int ldo, __nv_bfloat16* __restrict__ o_b, const float* __restrict__ w,
                                      const float* __restrict__ gate, int ldg, int H, int vdim, float eps, int M, int gate_act) {
    pdl_release();
    pdl_wait();
    const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (idx >= M * H) return;
    const int r = idx / H, h = idx - r * H;
    float* row = o + (size_t)r * ldo + (size_t)h * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss = fmaf(row[c], row[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32) {
        float y = row[c] * inv * (w ? w[c] : 1.f);
        if (gate) {
            const float gz = gate[(size_t)r * ldg + (size_t)h * vdim + c];
            y *= gate_act == 1 ? sigmoidf_(gz) : gate_act == 2 ? siluf_(gz) : gz;
        }
        row[c] = y;
        if (o_b) o_b[(size_t)r * ldo + (size_t)h * vdim + c] = __float2bfloat16_rn(y);
    }
}

// ---- launchers --------------------------------------------------------------------------------------------------------
cudaError_t launch_layernorm_rows(const float* x, const int* rows, const float* w, const float* b, float eps, float out_scale,
                                  float* out, void* out_bf16, int M, int D, cudaStream_t st, bool rms) {
    return launch_pdl(layernorm_rows_kernel, dim3(M), dim3(256), 0, st, x, rows, w, b, eps, out_scale, out,
                      reinterpret_cast<__nv_bfloat16*>(out_bf16), D, rms ? 1 : 0);
}

cudaError_t launch_pair_rows(const float* x, const float* x0, float* cat, void* cat_bf16, int M, int D, cudaStream_t st) {
    return launch_pdl(pair_rows_kernel, dim3(M), dim3(256), 0, st, x, x0, cat, reinterpret_cast<__nv_bfloat16*>(cat_bf16), D);
}

cudaError_t launch_add_rows(float* x, const float* y, int M, int D, cudaStream_t st) {
    const size_t n = (size_t)M * D;
    const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 8);
    return launch_pdl(add_rows_kernel, dim3(blocks), dim3(256), 0, st, x, y, n);
}

cudaError_t launch_xielu_rows(const float* proj, int ld, int off, float ap, float an, float* out, int ldo, int out_off,
                              void* out_bf16, int M, int F, cudaStream_t st, bool relu2) {
    return launch_pdl(xielu_rows_kernel, dim3(M, F > 1024 ? (F + 1023) / 1024 : 1), dim3(256), 0, st, proj, ld, off, ap, an, out,
                      ldo, out_off, reinterpret_cast<__nv_bfloat16*>(out_bf16), F, relu2 ? 1 : 0);
}

cudaError_t launch_talk_prep(float* proj, int ld, const float* bias, int q_off, int k_off, int v_off, int gate_off,
                             const TalkShape& a, const float* qw, const float* kw, float eps, float* kcache, float* vcache,
                             const PageMap& pm, const RowMeta& rm, int M, cudaStream_t st) {
    if (a.rot_dims % 2 || a.rot_dims > a.dim) return cudaErrorInvalidValue;
    return launch_pdl(talk_prep_kernel, dim3(M), dim3(256), 0, st, proj, ld, bias, q_off, k_off, v_off, gate_off, a.heads, a.kv_heads,
                      a.dim, a.vdim, qw, kw, eps, a.scale, a.rot_freq, a.rot_dims, kcache, vcache, pm.table, pm.max_pages,
                      pm.page_size, rm.slot, rm.pos);
}

static size_t talk_smem(const TalkShape& a, int TQ) {
    const int D4 = (a.dim + 3) / 4, DQ = 4 * D4 + 4, SV = (a.vdim + 3) & ~3, kvs = std::max(DQ, SV), np = a.heads * TQ;
    return ((size_t)np * DQ + 2 * (size_t)kTalkTK * kvs + 2 * (size_t)np * kTalkTK + 3 * (size_t)np + (size_t)a.heads * a.heads) * 4 +
           2 * (size_t)TQ * 4;
}

template <int VU, int NP, int NW>
static cudaError_t launch_talk_inst(const float* proj, int ld, int q_off, int gate_off, const float* kcache, const float* vcache,
                                    const PageMap& pm, const TalkShape& a, const RowMeta& rm, float* out, int ldo,
                                    __nv_bfloat16* out_b, float* part, unsigned* arrived, int M, int TQ, int S, cudaStream_t st) {
    const size_t smem = talk_smem(a, TQ);
    static size_t allowed[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || allowed[dev] < smem) {
        e = cudaFuncSetAttribute(talk_attention_kernel<VU, NP, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) allowed[dev] = smem;
    }
    return launch_pdl(talk_attention_kernel<VU, NP, NW>, dim3((M + TQ - 1) / TQ, S), dim3(NW * 32), smem, st, proj, ld, q_off,
                      gate_off, kcache, vcache, pm.table, pm.max_pages, pm.page_size, a.heads, a.kv_heads, a.dim, a.vdim, a.talk,
                      a.sink, rm.slot, rm.pos, out, ldo, out_b, M, TQ, part, arrived, a.window);
}

// the most pairs (heads x rows of a tile) a CTA carries: 128, 64 with values wider than 128 (accumulators per thread)
static int talk_max_pairs(int vdim) { return vdim > 128 ? 64 : 128; }

bool talk_attention_supported(const TalkShape& a) {
    return a.heads > 0 && a.kv_heads > 0 && a.heads % a.kv_heads == 0 && a.dim > 0 && a.vdim > 0 && a.vdim <= 256 &&
           a.heads <= talk_max_pairs(a.vdim) && talk_smem(a, 1) <= 200 * 1024;
}

// split_ws: kAttnRowsKernelMax * heads * kAttnSplitsMax * (vdim + 2) floats; arrived: kAttnRowsKernelMax zeroed counters.
// Prompt portions run 16 warps per CTA (up to 8 pairs per warp: half the accumulators of an 8-warp CTA, twice the warps
// to hide the latencies of a tile's dependent phases); a handful of rows run 8 warps per (row, share of the keys).
cudaError_t launch_talk_attention(const float* proj, int ld, int q_off, int gate_off, const float* kcache, const float* vcache,
                                  const PageMap& pm, const TalkShape& a, const RowMeta& rm, float* out, int ldo, void* out_bf16,
                                  float* split_ws, unsigned* arrived, int M, cudaStream_t st) {
    if (!talk_attention_supported(a)) return cudaErrorNotSupported;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(out_bf16);
    const int vu = (a.vdim + 31) / 32;
#define TALK_CASE(VU, NP, NW) \
    return launch_talk_inst<VU, NP, NW>(proj, ld, q_off, gate_off, kcache, vcache, pm, a, rm, out, ldo, ob, split_ws, arrived, M, TQ, S, st)
    if (M > kAttnRowsKernelMax) {
        int TQ = 16;
        const int S = 1;
        while (TQ > 1 && (a.heads * TQ > talk_max_pairs(a.vdim) || talk_smem(a, TQ) > 200 * 1024)) TQ >>= 1;
        if (vu <= 1) TALK_CASE(1, 8, 16);
        if (vu <= 2) TALK_CASE(2, 8, 16);
        if (vu <= 4) TALK_CASE(4, 8, 16);
        TALK_CASE(8, 4, 16);
    }
    // enough CTAs for two per SM, at least one key tile per share
    const int TQ = 1;
    const long long max_keys = (long long)pm.max_pages * pm.page_size;
    int S = (2 * 148 + M - 1) / M;
    S = (int)std::max<long long>(1, std::min<long long>(std::min(S, kAttnSplitsMax), (max_keys + kTalkTK - 1) / kTalkTK));
    const int np = (a.heads + 7) / 8;
    if (vu <= 1) { if (np <= 4) TALK_CASE(1, 4, 8); TALK_CASE(1, 16, 8); }
    if (vu <= 2) { if (np <= 4) TALK_CASE(2, 4, 8); TALK_CASE(2, 16, 8); }
    if (vu <= 4) { if (np <= 4) TALK_CASE(4, 4, 8); TALK_CASE(4, 16, 8); }
    if (np <= 4) TALK_CASE(8, 4, 8);
    TALK_CASE(8, 8, 8);
#undef TALK_CASE
}

cudaError_t launch_delta_prep(const float* proj, int ld, int beta_off, const DeltaShape& d, const float* tail, const RowMeta& rm,
                              float* rec, int ldr, int M, cudaStream_t st, int head_decay_off) {
    if (d.taps < 1 || d.taps > kMaxTaps) return cudaErrorNotSupported;
    const int C = 2 * d.kv_heads * d.dim + d.heads * d.vdim;
    const size_t smem = (size_t)C * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl(delta_prep_kernel, dim3(M), dim3(256), smem, st, proj, ld, beta_off, d.heads, d.kv_heads, d.dim, d.vdim, d.taps,
                      d.conv_w, tail, d.a_log, d.dt_bias, d.unit_eps, rm.slot, rm.pos, rm.start, rec, ldr, head_decay_off);
}

cudaError_t launch_conv_tail(const float* proj, int ld, int C, int taps, float* tail, const SeqMeta& sm, int n_seq,
                             cudaStream_t st) {
    if (taps <= 1) return cudaSuccess;
    return launch_pdl(conv_tail_kernel, dim3(n_seq, (C + 127) / 128), dim3(128), 0, st, proj, ld, C, taps, tail, sm.slot, sm.row0,
                      sm.count);
}

template <int RP, bool DELTA>
static cudaError_t launch_scan_inst(const float* in, int ld, const ScanInputs& si, int H, int G, int dim, int vdim, float* state,
                                    const SeqMeta& sm, const RowMeta& rm, int n_seq, float* o, int ldo, cudaStream_t st,
                                    bool head_decay, bool early) {
    const size_t smem = (size_t)((DELTA ? 3 : 2) * kScanTT * 8 * RP + kScanTT * kScanCols + kScanTT) * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(column_scan_kernel<RP, DELTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl_if(early, column_scan_kernel<RP, DELTA>, dim3(n_seq, H, (vdim + kScanCols - 1) / kScanCols), dim3(kScanThreads), smem, st,
                      in, ld, si.q_off, si.k_off, si.a_off, si.v_off, si.beta_off, H, G, dim, vdim, state, sm.slot, sm.row0,
                      sm.count, rm.pos, o, ldo, head_decay ? 1 : 0);
}

cudaError_t launch_gate_prep(float* proj, int ld, int q_off, int f_off, int v_off, const float* bias, const float* lower, int n_qf,
                             int n_v, int M, cudaStream_t st) {
    return launch_pdl(gate_prep_kernel, dim3(M), dim3(256), 0, st, proj, ld, q_off, f_off, v_off, bias, lower, n_qf, n_v);
}

// delta: the delta rule (reads k and beta); otherwise the gate-tied write (its inputs prepared by launch_gate_prep)
cudaError_t launch_column_scan(const float* in, int ld, const ScanInputs& si, bool delta, int H, int G, int dim, int vdim,
                               float* state, const SeqMeta& sm, const RowMeta& rm, int n_seq, float* o, int ldo,
                               cudaStream_t st, bool head_decay, bool early) {
    if (dim > 256 || H % G || H > 65535) return cudaErrorNotSupported;
#define SCAN_CASE(RP)                                                                                                    \
    return delta ? launch_scan_inst<RP, true>(in, ld, si, H, G, dim, vdim, state, sm, rm, n_seq, o, ldo, st, head_decay, early) \
                 : launch_scan_inst<RP, false>(in, ld, si, H, G, dim, vdim, state, sm, rm, n_seq, o, ldo, st, head_decay, early)
    if (dim <= 32) SCAN_CASE(4);
    if (dim <= 64) SCAN_CASE(8);
    if (dim <= 128) SCAN_CASE(16);
    SCAN_CASE(32);
#undef SCAN_CASE
}

template <int RP>
static cudaError_t launch_scalar_scan_inst(const float* in, int ld, const ScanInputs& si, int H, int dim, int vdim, float* state,
                                           const SeqMeta& sm, const RowMeta& rm, int n_seq, float* o, int ldo, cudaStream_t st,
                                           const float* fixed_decay, bool normaliser, bool early) {
    const size_t smem = (size_t)(2 * kScanTT * 8 * RP + kScanTT * kScanCols + 2 * kScanTT) * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(scalar_gate_scan_kernel<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl_if(early, scalar_gate_scan_kernel<RP>, dim3(n_seq, H, (vdim + (normaliser ? 1 : 0) + kScanCols - 1) / kScanCols),
                      dim3(kScanThreads), smem, st, in, ld, si.q_off, si.k_off, si.a_off, si.v_off, si.beta_off, H, dim, vdim, state,
                      sm.slot, sm.row0, sm.count, rm.pos, o, ldo, fixed_decay, normaliser ? 1 : 0);
}

cudaError_t launch_scalar_gate_scan(const float* in, int ld, const ScanInputs& si, int H, int dim, int vdim, float* state,
                                    const SeqMeta& sm, const RowMeta& rm, int n_seq, float* o, int ldo, cudaStream_t st,
                                    const float* fixed_decay, bool normaliser, bool early) {
    if (dim > 256 || H > 65535) return cudaErrorNotSupported;
    if (dim <= 32) return launch_scalar_scan_inst<4>(in, ld, si, H, dim, vdim, state, sm, rm, n_seq, o, ldo, st, fixed_decay, normaliser, early);
    if (dim <= 64) return launch_scalar_scan_inst<8>(in, ld, si, H, dim, vdim, state, sm, rm, n_seq, o, ldo, st, fixed_decay, normaliser, early);
    if (dim <= 128) return launch_scalar_scan_inst<16>(in, ld, si, H, dim, vdim, state, sm, rm, n_seq, o, ldo, st, fixed_decay, normaliser, early);
    return launch_scalar_scan_inst<32>(in, ld, si, H, dim, vdim, state, sm, rm, n_seq, o, ldo, st, fixed_decay, normaliser, early);
}

cudaError_t launch_head_norm_gate(float* o, int ldo, void* o_bf16, const float* w, const float* gate, int ldg, int H, int vdim,
                                  float eps, int M, cudaStream_t st, int gate_act) {
    return launch_pdl(head_norm_gate_kernel, dim3((M * H + 7) / 8), dim3(256), 0, st, o, ldo, reinterpret_cast<__nv_bfloat16*>(o_bf16),
                      w, gate, ldg, H, vdim, eps, M, gate_act);
}

}  // namespace lm

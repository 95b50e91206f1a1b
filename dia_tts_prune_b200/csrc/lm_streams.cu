// lm_streams.cu - kernels of the stream layer form of the language-model path (sm_100a): pre-norm sublayers over several
// residual streams (hyper-connections), attention over a cached latent, and the gates of a stabilised matrix memory.
//
// Same step layout and the same rule as lm_kernels.cu: every kernel computes a row's result from that row and the
// sequence state it points at, in an order of operations that does not depend on what else is in the batch.  The
// streams, norms, latents, scores, gates, running maxima and the recurrent state are fp32.
//
//   streams_embed_kernel      token rows of a bf16 table times a constant (optionally through an RMS norm), copied into every
//                             stream
//   streams_step_kernel       the write of one sublayer fused with the read of the next:  x_j <- sum_s mix[s][j] x_s +
//                             out[j] y (y: the sublayer's output, with the weighted sum of a row's expert outputs added),
//                             then u = sum_s in[s] x_s and h = layernorm(u) w, fp32 and the bf16 GEMM operand.  Without a
//                             write it is the first read of a step; without in / w it is the plain sum of the streams
//                             Options: a second output written with its own weights (a record whose sublayers read the same
//                             streams), a second norm weight on the same statistics, RMS instead of layer norm, the input
//                             row for assignments without a slot (identity experts), a sigmoid gate number on y
//   latent_prep_kernel        RMS norms of the query latent (in place, + bf16 operand) and of the key/value latent (into
//                             the pages: the latent is all an attention layer of this kind caches - and, behind it, one
//                             key part turned with the position where the layer has one)
//   rot_rows_kernel           rotary positions on a slice of every head of a row (pairs (2i, 2i + 1) or (i, i + dims / 2)),
//                             with a multiplier per group of heads, in place or into another buffer
//   latent_attention_rows_kernel  attention over the latent pages for shapes the tiled kernel does not take
//   head_linear_*_kernel      per-head products Y[m][h] = alpha A[m][h] . W[h]^T with an optional sigmoid gate: queries
//                             into the latent space (q_h^T W_uk,h) and attended latents out of it (W_uv,h o_h)
//   mlstm_gates_kernel        capped log-space input / forget gates and the running maximum m along a sequence's rows (a
//                             max-plus warp scan) -> decay exp(f + m' - m), write strength exp(i - m), floor exp(-m)
//   mlstm_finish_kernel       read-out / (max(|n . q|, floor) + 1e-6), per-head RMS norm, weight, sigmoid gate
//
// The attention itself is talk_attention_kernel of lm_mixers.cu with ONE key/value head whose key and value pages are
// the same latent pages (keys = values = c, head size = latent size), and the recurrence is scalar_gate_scan_kernel.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "lm_device.cuh"
#include "lm_internal.h"

namespace lm {

constexpr int kMaxStreams = 8;

// ---------------------------------------------------------------------------------------------------------------------
__global__ void streams_embed_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids, float scale,
                                     const float* __restrict__ norm_w, float eps, float* __restrict__ X, int streams, int V, int D) {
    __shared__ float red[32];
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x;
    const int id = ids[r];
    const bool ok = id >= 0 && id < V;
    float inv = 1.f;
    if (norm_w) {                                             // x / sqrt(mean(x^2) + eps) * w on the scaled row
        float ss = 0.f;
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            const float v = ok ? bf(table[(size_t)id * D + c]) * scale : 0.f;
            ss = fmaf(v, v, ss);
        }
        inv = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float v = ok ? bf(table[(size_t)id * D + c]) * scale : 0.f;
        if (norm_w) v = v * inv * norm_w[c];
        for (int j = 0; j < streams; ++j) X[((size_t)r * streams + j) * D + c] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// One CTA per (output) row.  X [M][S][D].  VW = 4: D is a multiple of 4 and every row is moved in 16-byte pieces.  The
// number of streams is a template argument, so that the old and new values of a column are exactly S registers each.
template <int VW, int S>
__global__ void __launch_bounds__(256)
streams_step_kernel(float* __restrict__ X, const float* __restrict__ mix, const float* __restrict__ out,
                    const float* __restrict__ y, const float* __restrict__ parts, const int* __restrict__ slot_of,
                    const float* __restrict__ sel_w, int top, const float* __restrict__ in, const float* __restrict__ norm_w,
                    float eps, const int* __restrict__ rows, float* __restrict__ h, __nv_bfloat16* __restrict__ h_b, int D,
                    const StreamExtra ex) {
    extern __shared__ __align__(16) float u_s[];              // [D]
    __shared__ float red[32];
    __shared__ float mix_s[S * S], out_s[S], in_s[S], out2_s[S];
    pdl_release();
    constexpr int s = S;
    const int tid = threadIdx.x;
    const bool write = (mix != nullptr) && !rows;
    if (tid < s * s) mix_s[tid] = write ? mix[tid] : 0.f;
    if (tid < s) {
        out_s[tid] = write ? out[tid] : 0.f;
        out2_s[tid] = (write && ex.y2) ? ex.out2[tid] : 0.f;
        in_s[tid] = in ? in[tid] : 1.f;
    }
    pdl_wait();
    __syncthreads();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = X + (size_t)r * s * D;
    auto load = [](const float* p, float (&v)[VW]) {
        if (VW == 4) {
            const float4 t = *reinterpret_cast<const float4*>(p);
            v[0] = t.x; v[1 % VW] = t.y; v[2 % VW] = t.z; v[3 % VW] = t.w;
        } else {
            v[0] = *p;
        }
    };
    auto store = [](float* p, const float (&v)[VW]) {
        if (VW == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1 % VW], v[2 % VW], v[3 % VW]);
        else *p = v[0];
    };
    float sum = 0.f;
    for (int c = tid * VW; c < D; c += blockDim.x * VW) {
        float xs[S][VW];
#pragma unroll
        for (int j = 0; j < S; ++j) {
            if (j < s) load(xr + (size_t)j * D + c, xs[j]);
            else
#pragma unroll
                for (int e = 0; e < VW; ++e) xs[j][e] = 0.f;
        }
        if (write) {
            float yv[VW];
#pragma unroll
            for (int e = 0; e < VW; ++e) yv[e] = 0.f;
            if (y) load(y + (size_t)r * D + c, yv);
            if (ex.y_gate) {                                  // one gate number per row on the unit's output
                const float gt = sigmoidf_(ex.y_gate[(size_t)r * ex.y_gate_ld]);
#pragma unroll
                for (int e = 0; e < VW; ++e) yv[e] *= gt;
            }
            if (parts)
                for (int t = 0; t < top; ++t) {
                    float pv[VW];
                    const int slot = slot_of[(size_t)r * top + t];    // < 0: an identity expert, its output is the input row
                    load(slot >= 0 ? parts + (size_t)slot * D + c : ex.ident_h + (size_t)r * D + c, pv);
                    const float wt = sel_w[(size_t)r * top + t];
#pragma unroll
                    for (int e = 0; e < VW; ++e) yv[e] = fmaf(wt, pv[e], yv[e]);
                }
            float y2v[VW];
#pragma unroll
            for (int e = 0; e < VW; ++e) y2v[e] = 0.f;
            if (ex.y2) load(ex.y2 + (size_t)r * D + c, y2v);  // the other sublayer's output of a parallel record
            float nx[S][VW];
#pragma unroll
            for (int j = 0; j < S; ++j) {
#pragma unroll
                for (int e = 0; e < VW; ++e) nx[j][e] = 0.f;
                if (j < s) {
#pragma unroll
                    for (int i = 0; i < S; ++i)
                        if (i < s) {
                            const float mw = mix_s[i * s + j];
#pragma unroll
                            for (int e = 0; e < VW; ++e) nx[j][e] = fmaf(mw, xs[i][e], nx[j][e]);
                        }
#pragma unroll
                    for (int e = 0; e < VW; ++e) nx[j][e] = fmaf(out_s[j], yv[e], fmaf(out2_s[j], y2v[e], nx[j][e]));
                    store(xr + (size_t)j * D + c, nx[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < S; ++j)
#pragma unroll
                for (int e = 0; e < VW; ++e) xs[j][e] = nx[j][e];
        }
        if (h) {
            float uv[VW];
#pragma unroll
            for (int e = 0; e < VW; ++e) uv[e] = 0.f;
#pragma unroll
            for (int j = 0; j < S; ++j)
                if (j < s)
#pragma unroll
                    for (int e = 0; e < VW; ++e) uv[e] = fmaf(in_s[j], xs[j][e], uv[e]);
            store(u_s + c, uv);
#pragma unroll
            for (int e = 0; e < VW; ++e) sum += uv[e];
        }
    }
    if (!h) return;
    if (!norm_w) {                                            // the plain read (every thread re-reads what it wrote itself)
        for (int c = tid * VW; c < D; c += blockDim.x * VW)
#pragma unroll
            for (int e = 0; e < VW; ++e) {
                h[(size_t)blockIdx.x * D + c + e] = u_s[c + e];
                if (h_b) h_b[(size_t)blockIdx.x * D + c + e] = __float2bfloat16_rn(u_s[c + e]);
            }
        return;
    }
    const float total = block_sum(sum, red);
    const float mean = ex.rms ? 0.f : total / (float)D;       // the RMS norm takes no mean off
    float v = 0.f;
    for (int c = tid; c < D; c += blockDim.x) {
        const float d = u_s[c] - mean;
        v = fmaf(d, d, v);
    }
    const float inv = 1.0f / sqrtf(block_sum(v, red) / (float)D + eps);
    for (int c = tid; c < D; c += blockDim.x) {
        const float n = (u_s[c] - mean) * inv, o = n * norm_w[c];
        h[(size_t)blockIdx.x * D + c] = o;
        if (h_b) h_b[(size_t)blockIdx.x * D + c] = __float2bfloat16_rn(o);
        if (ex.norm_w2) {                                     // a second weight on the same statistics: the other sublayer's input
            const float o2 = n * ex.norm_w2[c];
            ex.h2[(size_t)blockIdx.x * D + c] = o2;
            if (ex.h2_b) reinterpret_cast<__nv_bfloat16*>(ex.h2_b)[(size_t)blockIdx.x * D + c] = __float2bfloat16_rn(o2);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// turns the pair (a, b) by angle pos * f
__device__ __forceinline__ void turn_pair(float& a, float& b, int pos, float f) {
    float sn, cs;
    sincosf((float)pos * f, &sn, &cs);
    const float ra = a * cs - b * sn, rb = b * cs + a * sn;
    a = ra;
    b = rb;
}
// the partner of channel c of a vector whose first rot_dims channels turn: pairs (2i, 2i + 1) or (i, i + rot_dims / 2);
// `first`: whether c is the pair's first member; `i`: the pair's index
__device__ __forceinline__ int rot_partner(int c, int rot_dims, int half_layout, bool& first, int& i) {
    if (half_layout) {
        const int hf = rot_dims >> 1;
        first = c < hf;
        i = first ? c : c - hf;
        return first ? c + hf : c - hf;
    }
    first = (c & 1) == 0;
    i = c >> 1;
    return first ? c + 1 : c - 1;
}

// One CTA per row.  pages: [page][page_size][kv_rank + rot.n]: the normed latent, then (rot.n > 0) the columns
// c_off + kv_rank .. of the row, not normed, their first rot.dims channels turned with the row's position.
__global__ void __launch_bounds__(256)
latent_prep_kernel(float* __restrict__ proj, int ld, int q_off, int q_rank, int c_off, int kv_rank, const float* __restrict__ qw,
                   const float* __restrict__ cw, float eps, __nv_bfloat16* __restrict__ cq_b, float* __restrict__ pages,
                   const int* __restrict__ table, int max_pages, int page_size, const int* __restrict__ row_slot,
                   const int* __restrict__ row_pos, const RotPart rot) {
    __shared__ float red[32];
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x;
    float* row = proj + (size_t)r * ld;
    float ss = 0.f;
    for (int c = tid; c < q_rank; c += blockDim.x) ss = fmaf(row[q_off + c], row[q_off + c], ss);
    const float qinv = 1.0f / sqrtf(block_sum(ss, red) / (float)q_rank + eps);
    for (int c = tid; c < q_rank; c += blockDim.x) {
        const float v = row[q_off + c] * qinv * qw[c];
        row[q_off + c] = v;
        if (cq_b) cq_b[(size_t)r * q_rank + c] = __float2bfloat16_rn(v);
    }
    ss = 0.f;
    for (int c = tid; c < kv_rank; c += blockDim.x) ss = fmaf(row[c_off + c], row[c_off + c], ss);
    const float cinv = 1.0f / sqrtf(block_sum(ss, red) / (float)kv_rank + eps);
    const int pos = row_pos[r];
    const int page = table[(size_t)row_slot[r] * max_pages + pos / page_size];
    float* dst = pages + ((size_t)page * page_size + pos % page_size) * (kv_rank + rot.n);
    for (int c = tid; c < kv_rank; c += blockDim.x) dst[c] = row[c_off + c] * cinv * cw[c];
    const float* kr = row + c_off + kv_rank;
    for (int c = tid; c < rot.n; c += blockDim.x) {
        float v = kr[c];
        if (c < rot.dims) {
            bool first;
            int i;
            const int o = rot_partner(c, rot.dims, rot.half_layout, first, i);
            float a = first ? v : kr[o], b = first ? kr[o] : v;
            turn_pair(a, b, pos, rot.freq[i]);
            v = first ? a : b;
        }
        dst[kv_rank + c] = v;
    }
}

// dst[r][d_off + h dhs + c] = scale_h * turned(src[r][s_off + h shs + c]), c < n, for H heads per row: the first rot.dims
// channels turn with the row's position, the others pass.  Heads below `split` take scale_a, the others scale_b.  In place
// when dst == src with equal strides (a thread owns both members of a pair).
__global__ void __launch_bounds__(256)
rot_rows_kernel(const float* __restrict__ src, int lds, int s_off, int shs, float* __restrict__ dst, int ldd, int d_off, int dhs,
                int H, int n, int rot_dims, int half_layout, const float* __restrict__ freq, int split, float scale_a,
                float scale_b, const int* __restrict__ row_pos) {
    extern __shared__ float trig[];                           // [rot_dims / 2] sines, then as many cosines: one pair of them per
    pdl_release();                                            // turning pair of the row, shared by all heads
    pdl_wait();
    const int r = blockIdx.x, pos = row_pos[r], np = rot_dims >> 1, per = np + (n - rot_dims);   // items per head
    for (int i = threadIdx.x; i < np; i += blockDim.x) sincosf((float)pos * freq[i], &trig[i], &trig[np + i]);
    __syncthreads();
    const float* in = src + (size_t)r * lds + s_off;
    float* out = dst + (size_t)r * ldd + d_off;
    for (int idx = threadIdx.x; idx < H * per; idx += blockDim.x) {
        const int h = idx / per, it = idx - h * per;
        const float sc = h < split ? scale_a : scale_b;
        const float* ih = in + (size_t)h * shs;
        float* oh = out + (size_t)h * dhs;
        if (it < np) {
            const int c0 = half_layout ? it : 2 * it, c1 = half_layout ? it + np : 2 * it + 1;
            const float a = ih[c0], b = ih[c1], sn = trig[it], cs = trig[np + it];
            oh[c0] = (a * cs - b * sn) * sc;
            oh[c1] = (b * cs + a * sn) * sc;
        } else {
            const int c = rot_dims + (it - np);
            oh[c] = ih[c] * sc;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention over the latent pages for shapes the tiled kernel does not take (latents wider than 256, more heads than a
// tile holds): one CTA per (row, head), keys dealt to the warps in turn, every warp keeps its own running maximum,
// denominator and weighted latent sum (lane l owns latent channels l, l + 32, ...), and the warps' shares are merged in
// their fixed order with the sink's term.  q [M][H][R] carries the score multiplier; out [M][H][R].
constexpr int kLatentPerLane = 32;                            // latent channels per lane: R <= 1024
constexpr int kLatentWarps = 8;

__global__ void __launch_bounds__(kLatentWarps * 32)
latent_attention_rows_kernel(const float* __restrict__ q, const float* __restrict__ pages, const int* __restrict__ table,
                             int max_pages, int page_size, int H, int R, int RK, int window, const float* __restrict__ sink,
                             const int* __restrict__ row_slot, const int* __restrict__ row_pos, float* __restrict__ out) {
    extern __shared__ float sm[];                             // q [RK] | per warp: sums [R], maximum, denominator
    float* qs = sm;
    float* part = sm + RK;
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = row_pos[r];
    const int* pg = table + (size_t)row_slot[r] * max_pages;
    for (int c = threadIdx.x; c < RK; c += blockDim.x) qs[c] = q[((size_t)r * H + h) * RK + c];
    __syncthreads();
    float acc[kLatentPerLane];
#pragma unroll
    for (int u = 0; u < kLatentPerLane; ++u) acc[u] = 0.f;
    float m = -CUDART_INF_F, l = 0.f;
    const int j_lo = window > 0 ? max(0, pos - window + 1) : 0;
    for (int j = j_lo + warp; j <= pos; j += kLatentWarps) {
        const float* c = pages + ((size_t)pg[j / page_size] * page_size + j % page_size) * RK;
        float cv[kLatentPerLane], sc = 0.f;
#pragma unroll
        for (int u = 0; u < kLatentPerLane; ++u) {            // keys are the RK channels, values the first R of them
            const int ch = lane + 32 * u;
            cv[u] = ch < RK ? c[ch] : 0.f;
            sc = fmaf(ch < RK ? qs[ch] : 0.f, cv[u], sc);
        }
        sc = warp_sum(sc);
        const float mn = fmaxf(m, sc), corr = expf(m - mn), p = expf(sc - mn);
        l = fmaf(l, corr, p);
#pragma unroll
        for (int u = 0; u < kLatentPerLane; ++u) acc[u] = fmaf(acc[u], corr, p * cv[u]);
        m = mn;
    }
    float* mine = part + (size_t)warp * (R + 2);
#pragma unroll
    for (int u = 0; u < kLatentPerLane; ++u)
        if (lane + 32 * u < R) mine[lane + 32 * u] = acc[u];
    if (lane == 0) { mine[R] = m; mine[R + 1] = l; }
    __syncthreads();
    const float sk = sink ? sink[h] : -CUDART_INF_F;
    float top = sk;
    for (int w = 0; w < kLatentWarps; ++w) top = fmaxf(top, part[(size_t)w * (R + 2) + R]);
    float den = sink ? expf(sk - top) : 0.f;
    for (int w = 0; w < kLatentWarps; ++w) {
        const float mw = part[(size_t)w * (R + 2) + R];
        if (mw != -CUDART_INF_F) den = fmaf(part[(size_t)w * (R + 2) + R + 1], expf(mw - top), den);
    }
    const float f = den > 0.f ? 1.0f / den : 0.f;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < kLatentWarps; ++w) {
            const float mw = part[(size_t)w * (R + 2) + R];
            if (mw != -CUDART_INF_F) o = fmaf(part[(size_t)w * (R + 2) + c], expf(mw - top), o);
        }
        out[((size_t)r * H + h) * R + c] = o * f;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Y[m][h N + n] = alpha * sum_k A[m][h K + k] W[h][n][k]  [* sigmoid(gate[m][h N + n])].  64 x 64 x 16 tiles of fp32 FMAs,
// blockIdx.z = head.
constexpr int HB = 64, HK = 16;

__global__ void __launch_bounds__(256)
head_linear_tile_kernel(const float* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, float* __restrict__ Y, int ldy,
                        __nv_bfloat16* __restrict__ Yb, int M, int N, int K, float alpha, const float* __restrict__ gate, int ldg,
                        int a_hs, int y_hs) {
    __shared__ __align__(16) float As[HK][HB + 4];
    __shared__ __align__(16) float Bs[HK][HB + 4];
    const int hd = blockIdx.z, m0 = blockIdx.y * HB, n0 = blockIdx.x * HB;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const float* arow = (m0 + lr < M) ? A + (size_t)(m0 + lr) * lda + (size_t)hd * a_hs : nullptr;
    const __nv_bfloat16* wrow = (n0 + lr < N) ? W + ((size_t)hd * N + n0 + lr) * K : nullptr;
    const bool a_vec = (lda % 4 == 0) && (K % 4 == 0) && (a_hs % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    const bool w_vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 7) == 0);
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HK) {
        float a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f};
        const int k = k0 + lk;
        if (arow) {
            if (a_vec && k + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(arow + k);
                a4[0] = v.x; a4[1] = v.y; a4[2] = v.z; a4[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) a4[i] = arow[k + i];
            }
        }
        if (wrow) {
            if (w_vec && k + 3 < K) {
                const uint2 v = *reinterpret_cast<const uint2*>(wrow + k);
                const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
                const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
                b4[0] = __low2float(p0); b4[1] = __high2float(p0); b4[2] = __low2float(p1); b4[3] = __high2float(p1);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) b4[i] = bf(wrow[k + i]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lr] = a4[i];
            Bs[lk + i][lr] = b4[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j] * alpha;
            if (gate) v *= sigmoidf_(gate[(size_t)m * ldg + (size_t)hd * N + n]);
            Y[(size_t)m * ldy + (size_t)hd * y_hs + n] = v;
            if (Yb) Yb[(size_t)m * ldy + (size_t)hd * y_hs + n] = __float2bfloat16_rn(v);
        }
    }
}

// the same for a handful of rows: one warp per output element, the weights stream once per row
__global__ void __launch_bounds__(256)
head_linear_rows_kernel(const float* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, float* __restrict__ Y, int ldy,
                        __nv_bfloat16* __restrict__ Yb, int H, int N, int K, float alpha, const float* __restrict__ gate, int ldg,
                        int a_hs, int y_hs) {
    pdl_release();
    const int m = blockIdx.y, lane = threadIdx.x & 31;
    const int col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (col >= H * N) return;
    const int hd = col / N;
    const __nv_bfloat16* wrow = W + (size_t)col * K;          // W[h][n][k] is row h N + n of a [H N][K] matrix
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (a_hs % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 7) == 0) &&
                     ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    uint2 w0 = make_uint2(0u, 0u);
    if (vec && lane * 4 < K) w0 = *reinterpret_cast<const uint2*>(wrow + lane * 4);
    pdl_wait();
    const float* arow = A + (size_t)m * lda + (size_t)hd * a_hs;
    float acc = 0.f;
    if (vec) {
        for (int k = lane * 4; k < K; k += 128) {
            const uint2 wv = k == lane * 4 ? w0 : *reinterpret_cast<const uint2*>(wrow + k);
            const float4 x = *reinterpret_cast<const float4*>(arow + k);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&wv);
            acc = fmaf(x.x, __low2float(p[0]), acc);
            acc = fmaf(x.y, __high2float(p[0]), acc);
            acc = fmaf(x.z, __low2float(p[1]), acc);
            acc = fmaf(x.w, __high2float(p[1]), acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(arow[k], bf(wrow[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        float v = acc * alpha;
        if (gate) v *= sigmoidf_(gate[(size_t)m * ldg + col]);
        const size_t at = (size_t)m * ldy + (size_t)hd * y_hs + (col - hd * N);
        Y[at] = v;
        if (Yb) Yb[at] = __float2bfloat16_rn(v);
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// One warp per (scheduled sequence, head), 32 rows at a time.  m_t = max(f_t + m_(t-1), i_t) composes: a run of rows acts
// on the incoming maximum as m -> max(F + m, I) with F the sum of its f and I = max over its rows of (i_t + the f after
// it), and two runs combine as (F1 + F2, max(I1 + F2, I2)) - an inclusive warp scan gives every row its own (F, I).
__device__ __forceinline__ float logsigmoidf_(float z) { return z < -20.f ? z : -log1pf(expf(-z)); }

__global__ void __launch_bounds__(256)
mlstm_gates_kernel(float* __restrict__ proj, int ld, int i_off, int f_off, const float* __restrict__ bias, float cap, int H,
                   float* __restrict__ m_state, const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                   const int* __restrict__ seq_count, const int* __restrict__ row_pos, float* __restrict__ floor_out) {
    pdl_release();
    pdl_wait();
    const int s = blockIdx.x, lane = threadIdx.x & 31, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= H) return;
    const int slot = seq_slot[s], row0 = seq_row0[s], n = seq_count[s], start = row_pos[row0];
    const float bi = bias ? bias[i_off + h] : 0.f, bfg = bias ? bias[f_off + h] : 0.f;
    float m_in = start > 0 ? m_state[(size_t)slot * H + h] : 0.f;     // the running maximum starts at 0 with the sequence
    for (int t0 = 0; t0 < n; t0 += 32) {
        const bool ok = t0 + lane < n;
        float* row = proj + (size_t)(row0 + t0 + (ok ? lane : 0)) * ld;
        float ig = -CUDART_INF_F, fg = 0.f;                   // beyond the last row: the identity (F = 0, I = -inf)
        if (ok) {
            ig = cap * tanhf((row[i_off + h] + bi) / cap);
            fg = logsigmoidf_(cap * tanhf((row[f_off + h] + bfg) / cap));
        }
        float F = fg, I = ig;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float Fl = __shfl_up_sync(0xffffffffu, F, o), Il = __shfl_up_sync(0xffffffffu, I, o);
            if (lane >= o) {
                I = fmaxf(Il + F, I);
                F = Fl + F;
            }
        }
        const float m = fmaxf(F + m_in, I);
        float m_prev = __shfl_up_sync(0xffffffffu, m, 1);
        if (lane == 0) m_prev = m_in;
        if (ok) {
            row[i_off + h] = expf(ig - m);                    // write strength
            row[f_off + h] = expf(fg + m_prev - m);           // decay
            floor_out[(size_t)(row0 + t0 + lane) * H + h] = expf(-m);
        }
        m_in = __shfl_sync(0xffffffffu, m, 31);               // (lanes beyond the last row carry it on unchanged)
    }
    if (lane == 0) m_state[(size_t)slot * H + h] = m_in;
}

// one warp per (row, head).  raw [M][H][vdim + 1]: the read-out and, in its last column, n . q
__global__ void __launch_bounds__(256)
mlstm_finish_kernel(const float* __restrict__ raw, int ldr, const float* __restrict__ floor_in, float scale,
                    const float* __restrict__ w, const float* __restrict__ gate, int ldg, float eps, float* __restrict__ out,
                    __nv_bfloat16* __restrict__ out_b, int M, int H, int vdim) {
    pdl_release();
    pdl_wait();
    const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (idx >= M * H) return;
    const int r = idx / H, h = idx - r * H;
    const float* src = raw + (size_t)r * ldr + (size_t)h * (vdim + 1);
    const float den = fmaxf(fabsf(src[vdim] * scale), floor_in[(size_t)r * H + h]) + 1e-6f;
    const float mult = scale / den;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) {
        const float v = src[c] * mult;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    const size_t base = (size_t)r * H * vdim + (size_t)h * vdim;
    for (int c = lane; c < vdim; c += 32) {
        float y = src[c] * mult * inv * w[(size_t)h * vdim + c];
        if (gate) y *= sigmoidf_(gate[(size_t)r * ldg + (size_t)h * vdim + c]);
        out[base + c] = y;
        if (out_b) out_b[base + c] = __float2bfloat16_rn(y);
    }
}

// ---- launchers --------------------------------------------------------------------------------------------------------
cudaError_t launch_streams_embed(const void* table, const int* ids, float scale, float* X, int streams, int M, int V, int D,
                                 cudaStream_t st, const float* norm_w, float eps) {
    return launch_pdl(streams_embed_kernel, dim3(M), dim3(128), 0, st, reinterpret_cast<const __nv_bfloat16*>(table), ids, scale,
                      norm_w, eps, X, streams, V, D);
}

cudaError_t launch_streams_step(float* X, int streams, const StreamWrite& wr, const float* in, const float* norm_w, float eps,
                                const int* rows, float* h, void* h_bf16, int M, int D, cudaStream_t st, const StreamExtra& ex) {
    if (streams < 1 || streams > kMaxStreams) return cudaErrorNotSupported;
    const size_t smem = (size_t)D * 4;
    auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = D % 4 == 0 && aligned(X) && aligned(wr.y) && aligned(wr.parts) && aligned(ex.y2) && aligned(ex.ident_h);
    using Kernel = void (*)(float*, const float*, const float*, const float*, const float*, const int*, const float*, int, const float*,
                            const float*, float, const int*, float*, __nv_bfloat16*, int, const StreamExtra);
    Kernel kernel = nullptr;
    switch (streams) {
#define STREAMS_CASE(S) case S: kernel = vec ? streams_step_kernel<4, S> : streams_step_kernel<1, S>; break
        STREAMS_CASE(1); STREAMS_CASE(2); STREAMS_CASE(3); STREAMS_CASE(4);
        STREAMS_CASE(5); STREAMS_CASE(6); STREAMS_CASE(7); STREAMS_CASE(8);
#undef STREAMS_CASE
    }
    static size_t allowed[2][64] = {};
    if (smem > 48 * 1024) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64 || allowed[vec][dev] < smem) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) allowed[vec][dev] = smem;
        }
    }
    return launch_pdl(kernel, dim3(M), dim3(256), smem, st, X, wr.mix, wr.out, wr.y, wr.parts, wr.slot_of, wr.sel_w, wr.top,
                      in, norm_w, eps, rows, h, reinterpret_cast<__nv_bfloat16*>(h_bf16), D, ex);
}

cudaError_t launch_latent_prep(float* proj, int ld, int q_off, int q_rank, int c_off, int kv_rank, const float* qw,
                               const float* cw, float eps, void* cq_bf16, float* pages, const PageMap& pm, const RowMeta& rm,
                               int M, cudaStream_t st, const RotPart& rot) {
    if (rot.n < 0 || rot.dims < 0 || rot.dims % 2 || rot.dims > rot.n || (rot.dims > 0 && !rot.freq)) return cudaErrorInvalidValue;
    return launch_pdl(latent_prep_kernel, dim3(M), dim3(256), 0, st, proj, ld, q_off, q_rank, c_off, kv_rank, qw, cw, eps,
                      reinterpret_cast<__nv_bfloat16*>(cq_bf16), pages, pm.table, pm.max_pages, pm.page_size, rm.slot, rm.pos, rot);
}

cudaError_t launch_rot_rows(const float* src, int lds, int s_off, int shs, float* dst, int ldd, int d_off, int dhs, int H, int n,
                            const RotPart& rot, int split, float scale_a, float scale_b, const RowMeta& rm, int M, cudaStream_t st) {
    if (rot.dims < 0 || rot.dims % 2 || rot.dims > n || (rot.dims > 0 && !rot.freq)) return cudaErrorInvalidValue;
    return launch_pdl(rot_rows_kernel, dim3(M), dim3(256), (size_t)rot.dims * sizeof(float), st, src, lds, s_off, shs, dst, ldd, d_off, dhs, H, n, rot.dims,
                      rot.half_layout, rot.freq, split, scale_a, scale_b, rm.pos);
}

bool latent_attention_rows_supported(int H, int R) { return H > 0 && H <= 65535 && R > 0 && R <= 32 * kLatentPerLane; }

cudaError_t launch_latent_attention_rows(const float* q, const float* pages, const PageMap& pm, int H, int R, const float* sink,
                                         const RowMeta& rm, float* out, int M, cudaStream_t st, int key_extra, int window) {
    const int RK = R + key_extra;
    if (!latent_attention_rows_supported(H, RK)) return cudaErrorNotSupported;
    const size_t smem = ((size_t)RK + (size_t)kLatentWarps * (R + 2)) * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_pdl(latent_attention_rows_kernel, dim3(M, H), dim3(kLatentWarps * 32), smem, st, q, pages, pm.table, pm.max_pages,
                      pm.page_size, H, R, RK, window, sink, rm.slot, rm.pos, out);
}

cudaError_t launch_head_linear(const float* A, int lda, const void* W, float* Y, int ldy, void* y_bf16, int M, int H, int N, int K,
                               float alpha, const float* gate, int ldg, cudaStream_t st, int a_hs, int y_hs) {
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(W);
    __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(y_bf16);
    if (a_hs <= 0) a_hs = K;                                  // heads adjacent in A and in Y unless strides are given
    if (y_hs <= 0) y_hs = N;
    if (M <= kRowsKernelMax)
        return launch_pdl(head_linear_rows_kernel, dim3((H * N + 7) / 8, M), dim3(256), 0, st, A, lda, w, Y, ldy, yb, H, N, K, alpha,
                          gate, ldg, a_hs, y_hs);
    if (H > 65535) return cudaErrorNotSupported;
    head_linear_tile_kernel<<<dim3((N + HB - 1) / HB, (M + HB - 1) / HB, H), 256, 0, st>>>(A, lda, w, Y, ldy, yb, M, N, K, alpha, gate,
                                                                                          ldg, a_hs, y_hs);
    return cudaGetLastError();
}

cudaError_t launch_mlstm_gates(float* proj, int ld, int i_off, int f_off, const float* bias, float cap, int H, float* m_state,
                               const SeqMeta& sm, const RowMeta& rm, int n_seq, float* floor_out, cudaStream_t st) {
    if (H > 8 * 65535) return cudaErrorNotSupported;
    return launch_pdl(mlstm_gates_kernel, dim3(n_seq, (H + 7) / 8), dim3(256), 0, st, proj, ld, i_off, f_off, bias, cap, H, m_state, sm.slot,
                      sm.row0, sm.count, rm.pos, floor_out);
}

cudaError_t launch_mlstm_finish(const float* raw, int ldr, const float* floor_in, float scale, const float* w, const float* gate,
                                int ldg, float eps, float* out, void* out_bf16, int M, int H, int vdim, cudaStream_t st) {
    return launch_pdl(mlstm_finish_kernel, dim3((M * H + 7) / 8), dim3(256), 0, st, raw, ldr, floor_in, scale, w, gate, ldg, eps,
                      out, reinterpret_cast<__nv_bfloat16*>(out_bf16), M, H, vdim);
}

}  // namespace lm

// lm_kernels.cu - row kernels of the decoder-only language-model path (sm_100a).
//
// A step of the language-model engine is a flat batch of M rows: the new tokens of every scheduled sequence, one row per
// token, each row carrying (sequence slot, position, position of the first row its sequence has in this step).  Prompt
// portions, single decoded tokens and mixed batches are the same launch sequence.  Every kernel here computes a row's
// result from that row (and the sequence state it points at) alone, in an order of operations that does not depend on
// which other rows are in the batch - so the value at a position does not depend on how the prompt was cut or batched.
// (The only thing the row count selects is which of the two linear kernels runs; they sum in different orders, so a
// position computed in a step of a few rows and in a long one agrees to rounding, and to the bit within either kind.)
//
// Precision: activations, the residual stream, norms, router, attention scores / weights and the K/V pages are fp32;
// matrices are bf16 in memory and multiplied with fp32 accumulation.
//
//   embed_rows_bf16_kernel     token rows of a bf16 table
//   dyt_tapmix_kernel          DynamicTanh norm fused with the causal per-channel tap mix (short convolution over time,
//                              identity added), previous inputs from the step itself or from the sequence's tail state
//   tapmix_tail_kernel         keeps the last taps-1 normed inputs of every scheduled sequence
//   linear_tile_kernel         Y = A . W^T, 64 x 64 x 16 tiles of fp32 FMAs, optional row gather / scale / per-tile expert
//   linear_rows_kernel         the same interface for a handful of rows: one warp per output element; optional
//                              DynamicTanh + residual-add epilogue
//   dyt_tapmix_seq_kernel      norm + tap mix + tail update in one launch for a handful of rows
//   gated_rows_kernel          silu(gate) * up inside the [gate | up] product of a handful of rows / assignments
//   down_combine_rows_kernel   down products of a row's experts and the shared expert, their sum, norm, residual add
//   router_rows_kernel         router logits, top experts, scores and the assignment maps of a handful of rows
//   qk_norm_cache_kernel       whole-projection RMS norm of q and k, raw k and normed k scattered into the paged cache
//   sink_attention_split_kernel   softmax attention over the pages for a handful of rows, split over
//                              the keys: per-head temperature, tanh cap, linear distance bias, a window that keeps the
//                              first tokens, and a value-less sink term in the denominator
//   sink_attention_tile_kernel the same for prompt portions: 64 queries share the key / value tiles (flash-style)
//   pack_rows_bf16_kernel      the expert-grouped, score-scaled bf16 operand of the tensor-core products
//   router_topk_kernel         the `top` best experts of every row (optional logit bias) with sigmoid scores or the softmax
//                              over the chosen
//   moe_group_kernel           groups (row, expert) assignments by expert, padded to the GEMM's row tile
//   silu_mul_kernel            the gated unit's activation on [gate | up] rows: silu(gate) * up, or the clamped form
//   residual_dyt_kernel        x += DynamicTanh(y [+ the row's expert outputs])
//   dyt_gather_kernel          DynamicTanh of selected rows (the rows whose logits are wanted)
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "lm_device.cuh"
#include "lm_internal.h"

namespace lm {


// ---------------------------------------------------------------------------------------------------------------------
__global__ void embed_rows_bf16_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                       float* __restrict__ out, int V, int D) {
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x;
    const int id = ids[r];
    const bool ok = id >= 0 && id < V;
    for (int c = threadIdx.x; c < D; c += blockDim.x) out[(size_t)r * D + c] = ok ? bf(table[(size_t)id * D + c]) : 0.f;
}

// ---------------------------------------------------------------------------------------------------------------------
// out[r][c] = n_r[c] + sum_j cw[c][j] * n_{r - (taps-1-j)}[c],  n = DynamicTanh(x) of the same sequence, zero before its
// start.  Positions before this step's first row of the sequence come from tail[slot][i] (position start - (taps-1) + i).
__global__ void dyt_tapmix_kernel(const float* __restrict__ x, const float* __restrict__ nw, const float* __restrict__ nb,
                                  float alpha, const float* __restrict__ cw, int taps, const float* __restrict__ tail,
                                  const int* __restrict__ row_slot, const int* __restrict__ row_pos,
                                  const int* __restrict__ row_start, float* __restrict__ out,
                                  __nv_bfloat16* __restrict__ out_b, int D) {
    const int r = blockIdx.x;
    const int slot = row_slot[r], pos = row_pos[r], start = row_start[r];
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < D; c += gridDim.y * blockDim.x) {
        const float w = nw[c], b = nb[c];
        const float cur = dyt(x[(size_t)r * D + c], alpha, w, b);
        float acc = cur;
        if (taps > 0) acc = fmaf(cw[(size_t)c * taps + taps - 1], cur, acc);
        for (int o = 1; o < taps; ++o) {
            const int p = pos - o;
            if (p < 0) break;
            float v;
            if (p >= start) v = dyt(x[(size_t)(r - o) * D + c], alpha, w, b);
            else v = tail[((size_t)slot * (taps - 1) + (p - (start - (taps - 1)))) * D + c];
            acc = fmaf(cw[(size_t)c * taps + taps - 1 - o], v, acc);
        }
        out[(size_t)r * D + c] = acc;
        if (out_b) out_b[(size_t)r * D + c] = __float2bfloat16_rn(acc);       // the tensor-core operand of the same row
    }
}

// tail[slot][i] <- normed input at position (start + count) - (taps-1) + i, for every scheduled sequence s:
// from this step's rows when that position is in the step, else the old tail shifted by `count`.
__global__ void tapmix_tail_kernel(const float* __restrict__ x, const float* __restrict__ nw, const float* __restrict__ nb,
                                   float alpha, int taps, float* __restrict__ tail, const int* __restrict__ seq_slot,
                                   const int* __restrict__ seq_row0, const int* __restrict__ seq_count, int D) {
    const int s = blockIdx.x, T1 = taps - 1;
    const int slot = seq_slot[s], row0 = seq_row0[s], n = seq_count[s];
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < D; c += gridDim.y * blockDim.x) {
        float keep[kMaxTaps];
        float* t = tail + (size_t)slot * T1 * D + c;
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) {
            if (i >= T1) break;
            const int q = n - T1 + i;                             // row of the step, if >= 0
            if (q >= 0) keep[i] = dyt(x[(size_t)(row0 + q) * D + c], alpha, nw[c], nb[c]);
            else keep[i] = t[(size_t)(i + n) * D];                // old tail entry i + n  (< T1 because q < 0)
        }
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) {
            if (i >= T1) break;
            t[(size_t)i * D] = keep[i];
        }
    }
}

// Both of the above in one launch for a step of a few rows: one thread per (scheduled sequence, channel) walks the
// sequence's rows in order with the last taps-1 normed inputs in registers, and leaves them as the new tail.  Same
// operations in the same order as dyt_tapmix_kernel, so the two give the same bits.
__global__ void dyt_tapmix_seq_kernel(const float* __restrict__ x, const float* __restrict__ nw, const float* __restrict__ nb,
                                      float alpha, const float* __restrict__ cw, int taps, float* __restrict__ tail,
                                      const int* __restrict__ seq_slot, const int* __restrict__ seq_row0,
                                      const int* __restrict__ seq_count, const int* __restrict__ row_pos,
                                      float* __restrict__ out, int D) {
    pdl_release();
    pdl_wait();
    const int s = blockIdx.x, T1 = taps > 0 ? taps - 1 : 0;
    const int slot = seq_slot[s], row0 = seq_row0[s], n = seq_count[s];
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < D; c += gridDim.y * blockDim.x) {
        const float w = nw[c], b = nb[c];
        float prev[kMaxTaps];                                 // prev[o - 1]: the normed input o positions back
        float* t = tail + (size_t)slot * T1 * D + c;
#pragma unroll
        for (int o = 1; o < kMaxTaps; ++o) {
            if (o > T1) break;
            prev[o - 1] = t[(size_t)(T1 - o) * D];
        }
        for (int q = 0; q < n; ++q) {
            const int pos = row_pos[row0 + q];
            const float cur = dyt(x[(size_t)(row0 + q) * D + c], alpha, w, b);
            float acc = cur;
            if (taps > 0) acc = fmaf(cw[(size_t)c * taps + taps - 1], cur, acc);
#pragma unroll
            for (int o = 1; o < kMaxTaps; ++o) {
                if (o > T1 || pos - o < 0) break;
                acc = fmaf(cw[(size_t)c * taps + taps - 1 - o], prev[o - 1], acc);
            }
            out[(size_t)(row0 + q) * D + c] = acc;
#pragma unroll
            for (int o = kMaxTaps - 1; o >= 2; --o)
                if (o <= T1) prev[o - 1] = prev[o - 2];
            if (T1 >= 1) prev[0] = cur;
        }
#pragma unroll
        for (int o = 1; o < kMaxTaps; ++o) {
            if (o > T1) break;
            t[(size_t)(T1 - o) * D] = prev[o - 1];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Y[a][n] = sum_k scale_a * A[src_a][k] * W_e[n][k].  Without the maps: src_a = a, scale 1, expert 0.  With them
// (expert groups): a indexes padded assignment slots, a_row[a] < 0 is padding, the expert of a tile is a_expert of its
// first slot.  n_slots (device) bounds the slots in use; the grid covers the host's upper bound.
constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
linear_tile_kernel(const float* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, long long w_expert_stride,
                   float* __restrict__ Y, int ldy, int M, int N, int K, const int* __restrict__ a_row,
                   const float* __restrict__ a_scale, const int* __restrict__ a_expert, const int* __restrict__ n_slots) {
    __shared__ __align__(16) float As[BK][BM + 4];
    __shared__ __align__(16) float Bs[BK][BN + 4];
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int m_end = n_slots ? min(M, *n_slots) : M;
    if (m0 >= m_end) return;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const __nv_bfloat16* Wb = W + (a_expert ? (size_t)a_expert[m0] * (size_t)w_expert_stride : 0);

    // this thread's load coordinates: row (tid / 4) of the tile, 4 consecutive k
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    int src = -1;
    float sc = 1.f;
    if (m0 + lr < m_end) {
        src = a_row ? a_row[m0 + lr] : m0 + lr;
        if (a_scale && src >= 0) sc = a_scale[m0 + lr];
    }
    const float* arow = src >= 0 ? A + (size_t)src * lda : nullptr;
    const __nv_bfloat16* wrow = (n0 + lr < N) ? Wb + (size_t)(n0 + lr) * K : nullptr;
    const bool a_vec = (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    const bool w_vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(Wb) & 7) == 0);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
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
            As[lk + i][lr] = a4[i] * sc;
            Bs[lk + i][lr] = b4[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
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
        const int a = m0 + ty * 4 + i;
        if (a >= m_end) continue;
        if (a_row && a_row[a] < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) Y[(size_t)a * ldy + n] = acc[i][j];
        }
    }
}

// ---- the row kernels: a step of a few rows (decoding).  One warp per output element; the weights stream once per row,
// 16 bytes per lane.  Their epilogues do what the next kernel of a long step would: the DynamicTanh + residual add, the
// gate, the sum over a row's experts.
// wait_first: the first weight loads go out before pdl_wait, the activations are read after it
__device__ __forceinline__ float warp_dot(const float* __restrict__ arow, const __nv_bfloat16* __restrict__ wrow, int K, int lda,
                                          float sc, int lane, bool wait_first = false) {
    float acc = 0.f;
    const bool vec = (K % 8 == 0) && (lda % 4 == 0) && ((reinterpret_cast<uintptr_t>(wrow) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(arow) & 15) == 0);
    if (vec) {
        // eight 16-byte weight loads per lane in flight before their products (the sum keeps its order: k ascending)
        for (int k0 = lane * 8; k0 < K; k0 += 2048) {
            uint4 wv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = k0 + 256 * u;
                wv[u] = k < K ? *reinterpret_cast<const uint4*>(wrow + k) : make_uint4(0u, 0u, 0u, 0u);
            }
            if (wait_first) { pdl_wait(); wait_first = false; }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int k = k0 + 256 * u;
                if (k >= K) break;
                const float4 x0 = *reinterpret_cast<const float4*>(arow + k);
                const float4 x1 = *reinterpret_cast<const float4*>(arow + k + 4);
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&wv[u]);
                acc = fmaf(x0.x * sc, __low2float(p[0]), acc);
                acc = fmaf(x0.y * sc, __high2float(p[0]), acc);
                acc = fmaf(x0.z * sc, __low2float(p[1]), acc);
                acc = fmaf(x0.w * sc, __high2float(p[1]), acc);
                acc = fmaf(x1.x * sc, __low2float(p[2]), acc);
                acc = fmaf(x1.y * sc, __high2float(p[2]), acc);
                acc = fmaf(x1.z * sc, __low2float(p[3]), acc);
                acc = fmaf(x1.w * sc, __high2float(p[3]), acc);
            }
        }
    } else {
        if (wait_first) pdl_wait();
        for (int k = lane; k < K; k += 32) acc = fmaf(arow[k] * sc, bf(wrow[k]), acc);
    }
    if (wait_first) pdl_wait();                               // (K == 0: nothing was loaded)
    return warp_sum(acc);
}

// The whole warp of output element (a, n): h[a][n] = tapmix(norm(x_new)) of the next sublayer and its tail update, for a
// row that is its sequence's only row in the step.  Lane o fetches the input o positions back and its tap; the sum runs
// in dyt_tapmix_seq_kernel's order, so both give the same bits.
__device__ __forceinline__ void tap_out_warp(const TapOut& t, int a, int n, int D, float x_new, int lane) {
    const float cur = dyt(x_new, t.alpha, t.nw[n], t.nb[n]);
    const int taps = t.cw ? t.taps : 0, T1 = taps > 0 ? taps - 1 : 0;
    float acc = cur;
    if (taps > 0) acc = fmaf(t.cw[(size_t)n * taps + taps - 1], cur, acc);
    if (T1 > 0) {
        const int pos = t.row_pos[a];
        float* tl = t.tail + (size_t)t.row_slot[a] * T1 * D + n;
        float prev = 0.f, w = 0.f;
        if (lane >= 1 && lane <= T1) {
            prev = tl[(size_t)(T1 - lane) * D];
            w = t.cw[(size_t)n * taps + taps - 1 - lane];
        }
        for (int o = 1; o <= T1; ++o) {
            const float po = __shfl_sync(0xffffffffu, prev, o), wo = __shfl_sync(0xffffffffu, w, o);
            if (pos - o >= 0) acc = fmaf(wo, po, acc);
        }
        __syncwarp();                                         // every lane has read its tail entry
        if (lane >= 1 && lane <= T1 && T1 - lane - 1 >= 0) tl[(size_t)(T1 - lane - 1) * D] = prev;
        if (lane == 0) tl[(size_t)(T1 - 1) * D] = cur;
    }
    if (lane == 0) t.h[(size_t)a * D + n] = acc;
}

// Y[a][n] = dot, or with res_x: res_x[a][n] += DynamicTanh(dot), += dot without a norm (the residual stream takes the
// sublayer's output)
__global__ void __launch_bounds__(256)
linear_rows_kernel(const float* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, long long w_expert_stride,
                   float* __restrict__ Y, int ldy, int M, int N, int K, const int* __restrict__ a_row,
                   const float* __restrict__ a_scale, const int* __restrict__ a_expert, const int* __restrict__ n_slots,
                   float* __restrict__ res_x, const float* __restrict__ nw, const float* __restrict__ nb, float alpha,
                   const TapOut next) {
    pdl_release();
    const bool mapped = a_row || a_scale || a_expert || n_slots;      // the maps are an earlier kernel's output
    if (mapped) pdl_wait();
    const int a = blockIdx.y;
    const int m_end = n_slots ? min(M, *n_slots) : M;
    if (a >= m_end) return;
    const int src = a_row ? a_row[a] : a;
    if (src < 0) return;
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    const float sc = a_scale ? a_scale[a] : 1.f;
    const __nv_bfloat16* wrow = W + (a_expert ? (size_t)a_expert[a] * (size_t)w_expert_stride : 0) + (size_t)n * K;
    const float acc = warp_dot(A + (size_t)src * lda, wrow, K, lda, sc, lane, !mapped);
    if (res_x) {
        const float x_new = res_x[(size_t)a * ldy + n] + (nw ? dyt(acc, alpha, nw[n], nb[n]) : acc);
        __syncwarp();                                         // all lanes have read the old value
        if (lane == 0) res_x[(size_t)a * ldy + n] = x_new;
        if (next.h) tap_out_warp(next, a, n, ldy, x_new, lane);
    } else if (lane == 0) {
        Y[(size_t)a * ldy + n] = acc;
    }
}

// mid[a][n] = act(A_a . Wg_e[n], A_a . Wu_e[n]) (silu(g) u, or the clamped form of glu_act),  W_e = [gate rows (F) | up rows
// (F)][K].  blockIdx.y < n_assign: the
// assignment slot a of the routed experts (row, expert and score from the maps); beyond: row blockIdx.y - n_assign through
// the shared expert Ws (Sf hidden units) into smid.  One grid for both, so that the two weight streams overlap.
__global__ void __launch_bounds__(256)
gated_rows_kernel(const float* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, long long w_expert_stride,
                  float* __restrict__ mid, int n_assign, int F, int K, const int* __restrict__ a_row,
                  const float* __restrict__ a_scale, const int* __restrict__ a_expert, const __nv_bfloat16* __restrict__ Ws,
                  float* __restrict__ smid, int Sf, const GluAct act) {
    pdl_release();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int a = blockIdx.y, src, width;
    float sc = 1.f;
    const __nv_bfloat16* wg;
    float* dst;
    const bool routed = a < n_assign;                         // the routed slots need the router's maps first
    if (routed) {
        pdl_wait();
        src = a_row ? a_row[a] : a;
        if (src < 0 || n >= F) return;
        if (a_scale) sc = a_scale[a];
        wg = W + (a_expert ? (size_t)a_expert[a] * (size_t)w_expert_stride : 0) + (size_t)n * K;
        width = F;
        dst = mid + (size_t)a * F + n;
    } else {
        a -= n_assign;
        if (n >= Sf) return;
        src = a;
        wg = Ws + (size_t)n * K;
        width = Sf;
        dst = smid + (size_t)a * Sf + n;
    }
    const float* arow = A + (size_t)src * lda;
    const float g = warp_dot(arow, wg, K, lda, sc, lane, !routed);
    const float u = warp_dot(arow, wg + (size_t)width * K, K, lda, sc, lane);
    if (lane == 0) *dst = glu_act(act.kind, g, u, routed ? act.limit : act.shared_limit);
}

// v = smid[r] . Wsd[n] (with a shared expert) + sum_t [a_weight[r * top + t]] mid[r * top + t] . Wd_{e(r, t)}[n];
// x[r][n] += DynamicTanh(v), or x[r][n] = v without a norm
__global__ void __launch_bounds__(256)
down_combine_rows_kernel(const float* __restrict__ mid, int F, const __nv_bfloat16* __restrict__ Wd, const int* __restrict__ a_expert,
                         int top, const float* __restrict__ smid, int Sf, const __nv_bfloat16* __restrict__ Wsd,
                         float* __restrict__ x, int D, const float* __restrict__ nw, const float* __restrict__ nb, float alpha,
                         const TapOut next, const float* __restrict__ a_weight, int n_real, const float* __restrict__ ident_h,
                         const float* __restrict__ shared_gate, int shared_gate_ld) {
    pdl_release();
    const int r = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= D) return;
    float v = 0.f;
    if (smid) {
        v = warp_dot(smid + (size_t)r * Sf, Wsd + (size_t)n * Sf, Sf, Sf, 1.f, lane, true);
        if (shared_gate) v *= sigmoidf_(shared_gate[(size_t)r * shared_gate_ld]);     // one gate number per row
    } else {
        pdl_wait();
    }
    for (int t = 0; t < top; ++t) {
        const int a = r * top + t;
        // an output beyond the n_real experts is an identity expert: its output is the row's input
        const float part = (ident_h && a_expert[a] >= n_real)
                               ? ident_h[(size_t)r * D + n]
                               : warp_dot(mid + (size_t)a * F, Wd + ((size_t)a_expert[a] * D + n) * F, F, F, 1.f, lane);
        v = a_weight ? fmaf(a_weight[a], part, v) : v + part;
    }
    if (nw) {
        const float x_new = x[(size_t)r * D + n] + dyt(v, alpha, nw[n], nb[n]);
        __syncwarp();                                         // all lanes have read the old value
        if (lane == 0) x[(size_t)r * D + n] = x_new;
        if (next.h) tap_out_warp(next, r, n, D, x_new, lane);
    } else if (lane == 0) {
        x[(size_t)r * D + n] = v;                             // no norm: the plain sum
    }
}

// Routing of one row by one warp under a GroupedRoute rule.  z [n]: the row's router logits.  scores = softmax(z) over all n
// outputs; choice scores = scores + correction; with groups, only outputs of the `keep` groups (of n / count neighbours)
// whose largest choice score is largest can be chosen (ties: the lower group, the lower output); the `top` largest choice
// scores are taken in descending order and weighed by their scores (without the correction), divided by their sum and
// times `scale`.  cs [n] and gs [count] are this warp's scratch in shared memory.  out_e / out_w [top].
__device__ void grouped_route_warp(const float* __restrict__ z, int n, int top, const GroupedRoute& g, float* cs, float* gs,
                                   int lane, int* __restrict__ out_e, float* __restrict__ out_w) {
    float m = -CUDART_INF_F;
    for (int e = lane; e < n; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float den = 0.f;
    for (int e = lane; e < n; e += 32) den += expf(z[e] - m);
    den = warp_sum(den);
    for (int e = lane; e < n; e += 32) cs[e] = expf(z[e] - m) / den + (g.correction ? g.correction[e] : 0.f);
    __syncwarp();
    if (g.count > 1 && g.keep < g.count) {
        const int size = n / g.count;
        for (int q = lane; q < g.count; q += 32) {
            float best = -CUDART_INF_F;
            for (int e = q * size; e < (q + 1) * size; ++e) best = fmaxf(best, cs[e]);
            gs[q] = best;
        }
        __syncwarp();
        for (int pass = 0; pass < g.keep; ++pass) {           // every lane finds the same group; kept groups are marked
            float best = -CUDART_INF_F;
            int bq = -1;
            for (int q = 0; q < g.count; ++q) {
                const float v = gs[q];
                if (v != CUDART_INF_F && (bq < 0 || v > best)) { best = v; bq = q; }
            }
            __syncwarp();
            if (lane == 0 && bq >= 0) gs[bq] = CUDART_INF_F;
            __syncwarp();
        }
        for (int e = lane; e < n; e += 32)
            if (gs[e / size] != CUDART_INF_F) cs[e] = -CUDART_INF_F;
        __syncwarp();
    }
    float sum = 0.f;
    for (int t = 0; t < top; ++t) {
        float best = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int e = lane; e < n; e += 32) {
            bool taken = false;
            for (int u = 0; u < t; ++u) taken |= (out_e[u] == e);
            const float v = cs[e];
            if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        const float sc = expf(z[bi] - m) / den;               // the score itself, as computed above
        sum += sc;
        if (lane == 0) { out_e[t] = bi; out_w[t] = sc; }
        __syncwarp();
    }
    if (lane == 0)
        for (int t = 0; t < top; ++t) out_w[t] = out_w[t] / (sum + 1e-20f) * g.scale;
    __syncwarp();
}

// One CTA per row: router logits z = h . Wr^T [+ bias] (fp32), the `top` largest in descending order (ties: the lower
// index), scores sigmoid(z) - or, with softmax_top, the softmax over the chosen logits alone - and the assignment maps of
// the row kernels: slot r * top + t holds (row r, expert, score).
__global__ void __launch_bounds__(256)
router_rows_kernel(const float* __restrict__ h, int D, const __nv_bfloat16* __restrict__ Wr, int E, int top,
                   float* __restrict__ z_out, int* __restrict__ a_row, float* __restrict__ a_scale, int* __restrict__ a_expert,
                   int* __restrict__ slot_of, int* __restrict__ n_slots, const float* __restrict__ bias, int softmax_top,
                   const GroupedRoute gr) {
    extern __shared__ float zs[];                             // [E] (+ [n] + [count] scratch of the grouped rule)
    pdl_release();
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (warp >= E) pdl_wait();                                // (a warp without an expert may still write the maps below)
    for (int e = warp; e < E; e += nwarp) {
        const float z = warp_dot(h + (size_t)r * D, Wr + (size_t)e * D, D, D, 1.f, lane, e == warp) + (bias ? bias[e] : 0.f);
        if (lane == 0) { zs[e] = z; z_out[(size_t)r * E + e] = z; }
    }
    __syncthreads();
    if (warp != 0) return;
    if (r == 0 && lane == 0) *n_slots = gridDim.x * top;
    if (gr.n > 0) {                                           // E = gr.n router outputs (+ the shared unit's gate row)
        grouped_route_warp(zs, gr.n, top, gr, zs + E, zs + E + gr.n, lane, a_expert + r * top, a_scale + r * top);
        if (lane == 0)
            for (int t = 0; t < top; ++t) {
                const int a = r * top + t;
                const bool real = a_expert[a] < gr.n_real;    // an identity expert has no products: no row, no slot
                a_row[a] = real ? r : -1;
                slot_of[a] = real ? a : -1;
            }
        return;
    }
    float first = 0.f, den = 0.f;                             // softmax over the chosen: the first is the largest
    for (int t = 0; t < top; ++t) {
        float best = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            bool taken = false;
            for (int u = 0; u < t; ++u) taken |= (a_expert[r * top + u] == e);
            const float v = zs[e];
            if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            const int a = r * top + t;
            a_row[a] = r;
            a_expert[a] = bi;
            if (t == 0) first = best;
            const float sc = softmax_top ? expf(best - first) : 1.0f / (1.0f + expf(-best));
            den += sc;
            a_scale[a] = sc;
            slot_of[a] = a;
        }
        __syncwarp();
    }
    if (softmax_top && lane == 0)
        for (int t = 0; t < top; ++t) a_scale[r * top + t] /= den;
}

// ---------------------------------------------------------------------------------------------------------------------
// qk rows are [q (nq) | k (nk)].  q <- q / rms(q) * qw in place; the raw k goes to the value pages, k / rms(k) * kw to the
// key pages.  Pages: [page][kv head][page_size][dim] per layer; the sequence's page j / page_size is table[slot][..].
__global__ void qk_norm_cache_kernel(float* __restrict__ qk, int nq, int nk, const float* __restrict__ qw,
                                     const float* __restrict__ kw, float eps, float* __restrict__ kcache,
                                     float* __restrict__ vcache, const int* __restrict__ table, int max_pages, int page_size,
                                     int kv_heads, int dim, const int* __restrict__ row_slot,
                                     const int* __restrict__ row_pos) {
    __shared__ float red[32];
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x;
    float* q = qk + (size_t)r * (nq + nk);
    float* k = q + nq;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) sq = fmaf(q[c], q[c], sq);
    for (int c = threadIdx.x; c < nk; c += blockDim.x) sk = fmaf(k[c], k[c], sk);
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float rq = 1.0f / sqrtf(sq / (float)nq + eps), rk = 1.0f / sqrtf(sk / (float)nk + eps);
    for (int c = threadIdx.x; c < nq; c += blockDim.x) q[c] = q[c] * rq * qw[c];
    const int pos = row_pos[r];
    const int page = table[(size_t)row_slot[r] * max_pages + pos / page_size], off = pos % page_size;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const int g = c / dim, d = c - g * dim;
        const size_t at = (((size_t)page * kv_heads + g) * page_size + off) * dim + d;
        const float raw = k[c];
        vcache[at] = raw;
        kcache[at] = raw * rk * kw[c];
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention of a few rows (decoding), split over the keys.  Query position i sees key j <= i when i - j < window or
// j < keep_first (window <= 0: every j <= i).  score = cap * tanh(q.k * scale * temp_h / cap) - slope_h * (i - j)
// (cap <= 0: no cap).  One CTA per (row, up to HG query heads of one key/value head, split of the visible keys): a warp
// takes every eighth key of the split, reads its key and value rows once for all HG heads (lanes over the head size,
// coalesced), and keeps a running (maximum, denominator, weighted value sum) per head; the CTA's warps are merged and
// written as one partial per (row, head, split).  The CTA that arrives last at its (row, head chunk) merges the splits in
// their fixed order and adds the sink: exp(sink_h) joins the denominator only (no key, no value).
constexpr int kSplitThreads = 256, kSplitWarps = kSplitThreads / 32;
constexpr int kAttnMaxDimPerLane = 8;                         // head dim <= 256

// merges the S partial results of each of the nh <= 4 heads h0 .. of row r in their fixed order and adds the sink; one
// CTA of at least 4 warps: warp w weighs the splits of head h0 + w, then all threads sum.  scratch: >= 4 * 33 floats
__device__ __forceinline__ void combine_splits(const float* __restrict__ part, int S, int heads, int dim,
                                               const float* __restrict__ sink, float* __restrict__ out,
                                               __nv_bfloat16* __restrict__ out_b, int r, int h0, int nh, float* scratch) {
    static_assert(kAttnSplitsMax <= 32, "one lane per split");
    const size_t stride = (size_t)(dim + 2);
    const float* src0 = part + (size_t)(r * heads + h0) * S * stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                                          // the scratch's previous use is over
    if (warp < nh) {
        const float* src = src0 + (size_t)warp * S * stride;
        float* wgt = scratch + warp * 33;                     // exp(m_s - m) per split, 0 for an empty one; [32] = 1 / l
        const float ms = lane < S ? __ldcg(src + lane * stride) : -CUDART_INF_F;
        const float ls = lane < S ? __ldcg(src + lane * stride + 1) : 0.f;
        const float sk = sink ? sink[h0 + warp] : -CUDART_INF_F;
        const float m = fmaxf(sk, warp_max(ms));
        const float w = ms == -CUDART_INF_F ? 0.f : expf(ms - m);
        float l = sink ? expf(sk - m) : 0.f;
        for (int t = 0; t < S; ++t) l += __shfl_sync(0xffffffffu, ls * w, t);
        wgt[lane] = lane < S ? w : 0.f;
        if (lane == 0) wgt[32] = l > 0.f ? 1.0f / l : 0.f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nh * dim; idx += blockDim.x) {
        const int hh = idx / dim, c = idx - hh * dim;
        const float* src = src0 + (size_t)hh * S * stride + 2 + c;
        const float* wgt = scratch + hh * 33;
        float o = 0.f;
#pragma unroll 8
        for (int s = 0; s < S; ++s) o = fmaf(__ldcg(src + s * stride), wgt[s], o);
        o *= wgt[32];
        out[((size_t)r * heads + h0 + hh) * dim + c] = o;
        if (out_b) out_b[((size_t)r * heads + h0 + hh) * dim + c] = __float2bfloat16_rn(o);
    }
}

template <int HG>
__global__ void __launch_bounds__(kSplitThreads)
sink_attention_split_kernel(const float* __restrict__ qk, int q_stride, const float* __restrict__ kcache,
                            const float* __restrict__ vcache, const int* __restrict__ table, int max_pages, int page_size,
                            int heads, int kv_heads, int dim, float scale, float cap, const float* __restrict__ temp,
                            const float* __restrict__ slopes, const float* __restrict__ sink, int window, int keep_first,
                            const int* __restrict__ row_slot, const int* __restrict__ row_pos, float* __restrict__ part,
                            unsigned* __restrict__ arrived, float* __restrict__ out, __nv_bfloat16* __restrict__ out_b) {
    __shared__ float sm_m[kSplitWarps][HG], sm_l[kSplitWarps][HG];
    __shared__ bool is_last;
    __shared__ float sm_acc[kSplitWarps][HG][32 * kAttnMaxDimPerLane];
    pdl_release();
    pdl_wait();
    const int r = blockIdx.x, S = gridDim.z, sp = blockIdx.z;
    const int group = heads / kv_heads, chunks = (group + HG - 1) / HG;
    const int g = blockIdx.y / chunks, h0 = g * group + (blockIdx.y % chunks) * HG;
    const int nh = min(HG, (g + 1) * group - h0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int i = row_pos[r];
    const int* pages = table + (size_t)row_slot[r] * max_pages;
    const int lo = window > 0 ? max(0, i - window + 1) : 0;
    const int n_keep = window > 0 ? min(keep_first, lo) : 0;
    const int n_keys = n_keep + (i - lo + 1);
    const int per = (n_keys + S - 1) / S;
    const int k_begin = sp * per, k_end = min(n_keys, k_begin + per);
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    float q[HG][kAttnMaxDimPerLane], acc[HG][kAttnMaxDimPerLane], m_run[HG], l_run[HG], mult[HG], slope[HG];
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
        const int h = h0 + min(hh, nh - 1);
        mult[hh] = scale * (temp ? temp[h] : 1.f);
        slope[hh] = slopes ? slopes[h] : 0.f;
        m_run[hh] = -CUDART_INF_F; l_run[hh] = 0.f;
#pragma unroll
        for (int u = 0; u < kAttnMaxDimPerLane; ++u) {
            const int c = lane + 32 * u;
            q[hh][u] = c < dim ? qk[(size_t)r * q_stride + (size_t)h * dim + c] : 0.f;
            acc[hh][u] = 0.f;
        }
    }
    // the next key's rows are requested before the current key's arithmetic (a warp's keys are a dependent chain)
    float kv[kAttnMaxDimPerLane], vv[kAttnMaxDimPerLane], kn[kAttnMaxDimPerLane], vn[kAttnMaxDimPerLane];
    auto fetch = [&](int kk, float* kd, float* vd) -> int {
        const int j = kk < n_keep ? kk : lo + (kk - n_keep);
        const size_t at = (((size_t)pages[j / page_size] * kv_heads + g) * page_size + (j % page_size)) * dim;
#pragma unroll
        for (int u = 0; u < kAttnMaxDimPerLane; ++u) {
            const int c = lane + 32 * u;
            kd[u] = c < dim ? kcache[at + c] : 0.f;
            vd[u] = c < dim ? vcache[at + c] : 0.f;
        }
        return j;
    };
    int j_next = 0;
    if (k_begin + warp < k_end) j_next = fetch(k_begin + warp, kn, vn);
    for (int kk = k_begin + warp; kk < k_end; kk += kSplitWarps) {
        const int j = j_next;
#pragma unroll
        for (int u = 0; u < kAttnMaxDimPerLane; ++u) { kv[u] = kn[u]; vv[u] = vn[u]; }
        if (kk + kSplitWarps < k_end) j_next = fetch(kk + kSplitWarps, kn, vn);
        const float dist = (float)(i - j);
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
            float d = 0.f;
#pragma unroll
            for (int u = 0; u < kAttnMaxDimPerLane; ++u) d = fmaf(q[hh][u], kv[u], d);
            float sc = warp_sum(d) * mult[hh];
            if (cap > 0.f) sc = cap * tanhf(sc * inv_cap);
            sc -= slope[hh] * dist;
            const float m_new = fmaxf(m_run[hh], sc);
            const float corr = expf(m_run[hh] - m_new);       // exp(-inf) = 0 at the first key
            const float p = expf(sc - m_new);
            l_run[hh] = l_run[hh] * corr + p;
            m_run[hh] = m_new;
#pragma unroll
            for (int u = 0; u < kAttnMaxDimPerLane; ++u) acc[hh][u] = fmaf(p, vv[u], acc[hh][u] * corr);
        }
    }
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
        if (lane == 0) { sm_m[warp][hh] = m_run[hh]; sm_l[warp][hh] = l_run[hh]; }
#pragma unroll
        for (int u = 0; u < kAttnMaxDimPerLane; ++u) sm_acc[warp][hh][lane + 32 * u] = acc[hh][u];
    }
    __syncthreads();
    // merge the warps (fixed order); part[((r * heads + h) * S + sp)] = {maximum, denominator, sums[dim]}
    for (int hh = 0; hh < nh; ++hh) {
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kSplitWarps; ++w) m = fmaxf(m, sm_m[w][hh]);
        float* dst = part + ((size_t)(r * heads + h0 + hh) * S + sp) * (dim + 2);
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < kSplitWarps; ++w) l += sm_m[w][hh] == -CUDART_INF_F ? 0.f : sm_l[w][hh] * expf(sm_m[w][hh] - m);
        if (tid == 0) { dst[0] = m; dst[1] = l; }
        for (int c = tid; c < dim; c += kSplitThreads) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < kSplitWarps; ++w) o += sm_m[w][hh] == -CUDART_INF_F ? 0.f : sm_acc[w][hh][c] * expf(sm_m[w][hh] - m);
            dst[2 + c] = o;
        }
    }
    // the split that arrives last at its (row, head chunk) merges all of them: no second launch.  The counter goes back
    // to zero for the next step.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned* cnt = arrived + (size_t)r * gridDim.y + blockIdx.y;
        const unsigned seen = atomicAdd(cnt, 1u);
        is_last = seen == (unsigned)S - 1u;
        if (is_last) *cnt = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    static_assert(HG <= kSplitWarps, "one warp per head in the merge");
    combine_splits(part, S, heads, dim, sink, out, out_b, r, h0, nh, sm_acc[0][0]);
}

// ---------------------------------------------------------------------------------------------------------------------
// The same attention for prompt portions: one CTA per (64 consecutive rows of the step, query head), flash-style - key
// and value tiles of 64 positions gathered from the pages into padded shared memory and shared by the 64 queries, 4 x 4
// score blocks per thread, online softmax whose running maximum starts at the sink.  The rows of a tile may belong to
// several sequences: a maximal run of rows with one slot and consecutive positions is a segment, the segments are
// walked one after the other, and a row's statistics move only while its own segment is walked.  A segment's keys are
// the kept first positions that lie in front of its window range, then the range from the first row's window start to
// the last row; the visibility rule is applied per (query, key) pair.  NC: the head size in chunks of 64.
constexpr int kTQ = 64, kTK = 64, kTileThreads = 256, kTPStride = 68;

template <int NC>
__global__ void __launch_bounds__(kTileThreads, 1)
sink_attention_tile_kernel(const float* __restrict__ qk, int q_stride, const float* __restrict__ kcache,
                           const float* __restrict__ vcache, const int* __restrict__ table, int max_pages, int page_size,
                           int heads, int kv_heads, int dim, float scale, float cap, const float* __restrict__ temp,
                           const float* __restrict__ slopes, const float* __restrict__ sink, int window, int keep_first,
                           const int* __restrict__ row_slot, const int* __restrict__ row_pos, float* __restrict__ out,
                           __nv_bfloat16* __restrict__ out_b, int M) {
    constexpr int DP = 64 * NC, QS = DP + 4, C4 = DP / 4;
    extern __shared__ __align__(16) float sm[];
    float* Qs = sm;                                           // [64][QS]
    float* Ks = Qs + kTQ * QS;                                // [64][QS]
    float* Vs = Ks + kTK * QS;                                // [64][DP]
    float* Ps = Vs + kTK * DP;                                // [64][68]
    int* s_slot = reinterpret_cast<int*>(Ps + kTQ * kTPStride);   // [64]
    int* s_pos = s_slot + kTQ;                                // [64]

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int r0 = (gridDim.x - 1 - blockIdx.x) * kTQ, h = blockIdx.y;    // later rows see more keys: they start first
    const int n_rows = min(kTQ, M - r0);
    const int g = h / (heads / kv_heads);
    const bool vec = (dim % 4) == 0 && (q_stride % 4) == 0;
    const float mult = scale * (temp ? temp[h] : 1.f);
    const float slope = slopes ? slopes[h] : 0.f;
    const float sink_h = sink ? sink[h] : -CUDART_INF_F;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    if (tid < kTQ) {
        s_slot[tid] = tid < n_rows ? row_slot[r0 + tid] : -1;
        s_pos[tid] = tid < n_rows ? row_pos[r0 + tid] : -1;
    }
    for (int i = tid; i < kTQ * C4; i += kTileThreads) {
        const int r = i / C4, c = (i - r * C4) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < n_rows && c < dim) {
            const float* src = qk + (size_t)(r0 + r) * q_stride + (size_t)h * dim + c;
            if (vec) v = *reinterpret_cast<const float4*>(src);
            else {
                v.x = src[0];
                if (c + 1 < dim) v.y = src[1];
                if (c + 2 < dim) v.z = src[2];
                if (c + 3 < dim) v.w = src[3];
            }
        }
        *reinterpret_cast<float4*>(Qs + r * QS + c) = v;
    }

    float m_run[4], l_run[4], o[4][4 * NC];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m_run[i] = sink_h; l_run[i] = 0.f;
#pragma unroll
        for (int j = 0; j < 4 * NC; ++j) o[i][j] = 0.f;
    }
    __syncthreads();

    int seg_a = 0;
    while (seg_a < n_rows) {
        int seg_b = seg_a + 1;
        while (seg_b < n_rows && s_slot[seg_b] == s_slot[seg_a] && s_pos[seg_b] == s_pos[seg_b - 1] + 1) ++seg_b;
        const int* pages = table + (size_t)s_slot[seg_a] * max_pages;
        const int p_first = s_pos[seg_a], p_last = s_pos[seg_b - 1];
        const int lo = window > 0 ? max(0, p_first - window + 1) : 0;
        const int n_keep = window > 0 ? min(keep_first, lo) : 0;
        for (int phase = 0; phase < 2; ++phase) {
            const int k_begin = phase == 0 ? 0 : lo, k_end = phase == 0 ? n_keep : p_last + 1;
            // Head sizes up to 128 keep the next key / value tile in registers while the current one is multiplied (the
            // gather's latency hides behind the arithmetic); larger heads have no registers to spare and load in place.
            constexpr bool kAhead = NC <= 2;
            constexpr int PF = kAhead ? kTK * C4 / kTileThreads : 1;
            float4 kreg[PF], vreg[PF];
            auto gather = [&](int j0, int it, float4& kk, float4& vv) {
                const int i = tid + it * kTileThreads;
                const int r = i / C4, c = (i - r * C4) * 4, j = j0 + r;
                kk = make_float4(0.f, 0.f, 0.f, 0.f);
                vv = kk;
                if (j < k_end && c < dim) {
                    const size_t at = (((size_t)pages[j / page_size] * kv_heads + g) * page_size + (j % page_size)) * dim + c;
                    if (vec) {
                        kk = *reinterpret_cast<const float4*>(kcache + at);
                        vv = *reinterpret_cast<const float4*>(vcache + at);
                    } else {
                        kk.x = kcache[at]; vv.x = vcache[at];
                        if (c + 1 < dim) { kk.y = kcache[at + 1]; vv.y = vcache[at + 1]; }
                        if (c + 2 < dim) { kk.z = kcache[at + 2]; vv.z = vcache[at + 2]; }
                        if (c + 3 < dim) { kk.w = kcache[at + 3]; vv.w = vcache[at + 3]; }
                    }
                }
            };
            auto put = [&](int it, const float4& kk, const float4& vv) {
                const int i = tid + it * kTileThreads;
                const int r = i / C4, c = (i - r * C4) * 4;
                *reinterpret_cast<float4*>(Ks + r * QS + c) = kk;
                *reinterpret_cast<float4*>(Vs + r * DP + c) = vv;
            };
            if (kAhead && k_begin < k_end) {
#pragma unroll
                for (int it = 0; it < PF; ++it) gather(k_begin, it, kreg[it], vreg[it]);
            }
            for (int j0 = k_begin; j0 < k_end; j0 += kTK) {
                __syncthreads();                              // the previous tile is consumed
                if (kAhead) {
#pragma unroll
                    for (int it = 0; it < PF; ++it) put(it, kreg[it], vreg[it]);
                } else {
                    for (int it = 0; it < kTK * C4 / kTileThreads; ++it) {
                        float4 kk, vv;
                        gather(j0, it, kk, vv);
                        put(it, kk, vv);
                    }
                }
                __syncthreads();
                if (kAhead && j0 + kTK < k_end) {
#pragma unroll
                    for (int it = 0; it < PF; ++it) gather(j0 + kTK, it, kreg[it], vreg[it]);
                }
                // ---- S = Q K^T: rows ty*4 + i, keys tx + 16 j ----
                float sc[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
#pragma unroll 4
                for (int d4 = 0; d4 < C4; ++d4) {
                    float4 qa[4], ka[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) qa[i] = *reinterpret_cast<const float4*>(Qs + (ty * 4 + i) * QS + d4 * 4);
#pragma unroll
                    for (int j = 0; j < 4; ++j) ka[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * QS + d4 * 4);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            sc[i][j] = fmaf(qa[i].x, ka[j].x, sc[i][j]);
                            sc[i][j] = fmaf(qa[i].y, ka[j].y, sc[i][j]);
                            sc[i][j] = fmaf(qa[i].z, ka[j].z, sc[i][j]);
                            sc[i][j] = fmaf(qa[i].w, ka[j].w, sc[i][j]);
                        }
                }
                // ---- temperature, cap, distance bias, visibility; online softmax over the 16 threads of a row ----
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = ty * 4 + i;
                    const bool live = row >= seg_a && row < seg_b;
                    const int qi = s_pos[row];
                    float mx = -CUDART_INF_F;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int key = j0 + tx + 16 * j;
                        const bool ok = live && key < k_end && key <= qi && (window <= 0 || qi - key < window || key < keep_first);
                        float v = sc[i][j] * mult;
                        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
                        v -= slope * (float)(qi - key);
                        sc[i][j] = ok ? v : -CUDART_INF_F;
                        mx = fmaxf(mx, sc[i][j]);
                    }
#pragma unroll
                    for (int w = 8; w >= 1; w >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));
                    const float m_new = fmaxf(m_run[i], mx);
                    float corr = 1.f, psum = 0.f;
                    if (m_new == -CUDART_INF_F) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
                    } else {
                        corr = expf(m_run[i] - m_new);        // exp(-inf) = 0 on the first live tile without a sink
#pragma unroll
                        for (int j = 0; j < 4; ++j) { sc[i][j] = expf(sc[i][j] - m_new); psum += sc[i][j]; }
                    }
#pragma unroll
                    for (int w = 8; w >= 1; w >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, w);
                    l_run[i] = l_run[i] * corr + psum;
                    m_run[i] = m_new;
#pragma unroll
                    for (int j = 0; j < 4 * NC; ++j) o[i][j] *= corr;
#pragma unroll
                    for (int j = 0; j < 4; ++j) Ps[row * kTPStride + tx + 16 * j] = sc[i][j];
                }
                __syncthreads();
                // ---- O += P V: rows ty*4 + i, value columns 64 c + tx*4 .. +3 ----
#pragma unroll 2
                for (int c4 = 0; c4 < kTK / 4; ++c4) {
                    float4 pa[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) pa[i] = *reinterpret_cast<const float4*>(Ps + (ty * 4 + i) * kTPStride + c4 * 4);
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            const float4 v4 = *reinterpret_cast<const float4*>(Vs + (c4 * 4 + cc) * DP + 64 * c + tx * 4);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float pv = cc == 0 ? pa[i].x : cc == 1 ? pa[i].y : cc == 2 ? pa[i].z : pa[i].w;
                                o[i][4 * c + 0] = fmaf(pv, v4.x, o[i][4 * c + 0]);
                                o[i][4 * c + 1] = fmaf(pv, v4.y, o[i][4 * c + 1]);
                                o[i][4 * c + 2] = fmaf(pv, v4.z, o[i][4 * c + 2]);
                                o[i][4 * c + 3] = fmaf(pv, v4.w, o[i][4 * c + 3]);
                            }
                        }
                    }
                }
            }
        }
        seg_a = seg_b;
    }
    // ---- the sink's own term joins the denominator; normalise and store ----
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = ty * 4 + i;
        if (row >= n_rows) continue;
        float l = l_run[i];
        if (sink) l += expf(sink_h - m_run[i]);
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        const size_t base = ((size_t)(r0 + row) * heads + h) * dim;
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int col = 64 * c + tx * 4 + u;
                if (col < dim) {
                    const float v = o[i][4 * c + u] * inv;
                    out[base + col] = v;
                    if (out_b) out_b[base + col] = __float2bfloat16_rn(v);
                }
            }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// one warp per row: the `top` largest of z [+ bias] (ties: the lower index) in descending order; scores sigmoid(z), or
// with softmax_top the softmax over the chosen logits alone
__global__ void router_topk_kernel(const float* __restrict__ z, int E, int top, int M, int* __restrict__ sel_e,
                                   float* __restrict__ sel_w, const float* __restrict__ bias, int softmax_top,
                                   const GroupedRoute gr) {
    extern __shared__ float route_scratch[];                  // grouped rule: [warps][n + count]
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= M) return;
    const float* zr = z + (size_t)r * E;
    if (gr.n > 0) {                                           // rows of z are E = gr.n (+ 1) wide
        float* cs = route_scratch + (size_t)(threadIdx.x >> 5) * (gr.n + gr.count);
        grouped_route_warp(zr, gr.n, top, gr, cs, cs + gr.n, lane, sel_e + (size_t)r * top, sel_w + (size_t)r * top);
        return;
    }
    float first = 0.f, den = 0.f;
    for (int t = 0; t < top; ++t) {
        float best = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            bool taken = false;
            for (int u = 0; u < t; ++u) taken |= (sel_e[(size_t)r * top + u] == e);
            const float v = zr[e] + (bias ? bias[e] : 0.f);
            if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            sel_e[(size_t)r * top + t] = bi;
            if (t == 0) first = best;
            const float sc = softmax_top ? expf(best - first) : 1.0f / (1.0f + expf(-best));
            den += sc;
            sel_w[(size_t)r * top + t] = sc;
        }
        __syncwarp();
    }
    if (softmax_top && lane == 0)
        for (int t = 0; t < top; ++t) sel_w[(size_t)r * top + t] /= den;
}

// one CTA: counts per expert, group starts padded to `pad` slots, then a_row / a_scale / a_expert per slot and the slot
// of every assignment.  The order inside a group does not matter: every slot's row is computed on its own.
__global__ void moe_group_kernel(const int* __restrict__ sel_e, const float* __restrict__ sel_w, int n_assign, int top,
                                 int E, int pad, int* __restrict__ a_row, float* __restrict__ a_scale,
                                 int* __restrict__ a_expert, int* __restrict__ slot_of, int* __restrict__ n_slots,
                                 int max_slots) {
    extern __shared__ int sh[];
    int* count = sh;            // [E]
    int* start = sh + E;        // [E]
    int* cursor = sh + 2 * E;   // [E]
    for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int a = threadIdx.x; a < n_assign; a += blockDim.x)  // (an output beyond the E experts has no products: no slot)
        if (sel_e[a] < E) atomicAdd(&count[sel_e[a]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) { start[e] = at; at += (count[e] + pad - 1) / pad * pad; }
        *n_slots = at;
    }
    __syncthreads();
    const int total = min(*n_slots, max_slots);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int end = (e + 1 < E) ? start[e + 1] : total;
        for (int s = start[e]; s < end; ++s) { a_row[s] = -1; a_scale[s] = 0.f; a_expert[s] = e; }
    }
    __syncthreads();
    for (int a = threadIdx.x; a < n_assign; a += blockDim.x) {
        const int e = sel_e[a];
        if (e >= E) { slot_of[a] = -1; continue; }
        const int s = start[e] + atomicAdd(&cursor[e], 1);
        a_row[s] = a / top;
        a_scale[s] = sel_w[a];
        slot_of[a] = s;
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// mid (fp32) or mid_b (bf16, the operand of a tensor-core product: padding rows are written too, as zeros)
__global__ void silu_mul_kernel(const float* __restrict__ gu, float* __restrict__ mid, __nv_bfloat16* __restrict__ mid_b, int F,
                                const int* __restrict__ a_row, const int* __restrict__ n_slots, int M, int act, float limit) {
    const int a = blockIdx.x;
    if (n_slots && a >= min(M, *n_slots)) return;
    const bool pad = a_row && a_row[a] < 0;
    if (pad && !mid_b) return;
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
        float v = 0.f;
        if (!pad) {
            const float g = gu[(size_t)a * 2 * F + c], u = gu[(size_t)a * 2 * F + F + c];
            v = glu_act(act, g, u, limit);
        }
        if (mid_b) mid_b[(size_t)a * F + c] = __float2bfloat16_rn(v);
        else mid[(size_t)a * F + c] = v;
    }
}

// Ab[a] = bf16(scale_a * A[src_a]) for the assignment slots in use, zeros for padding slots: the expert-grouped operand
__global__ void pack_rows_bf16_kernel(const float* __restrict__ A, __nv_bfloat16* __restrict__ Ab, int D,
                                      const int* __restrict__ a_row, const float* __restrict__ a_scale,
                                      const int* __restrict__ n_slots, int M) {
    const int a = blockIdx.x;
    if (n_slots && a >= min(M, *n_slots)) return;
    const int src = a_row ? a_row[a] : a;
    const float sc = (a_scale && src >= 0) ? a_scale[a] : 1.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x)
        Ab[(size_t)a * D + c] = __float2bfloat16_rn(src >= 0 ? A[(size_t)src * D + c] * sc : 0.f);
}

// x[r] += DynamicTanh(y[r] + sum_t parts[slot_of[r * top + t]])   (y or parts may be absent)
__global__ void residual_dyt_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ parts,
                                    const int* __restrict__ slot_of, int top, const float* __restrict__ nw,
                                    const float* __restrict__ nb, float alpha, int D) {
    const int r = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < D; c += gridDim.y * blockDim.x) {
        float v = y ? y[(size_t)r * D + c] : 0.f;
        if (parts)
            for (int t = 0; t < top; ++t) v += parts[(size_t)slot_of[(size_t)r * top + t] * D + c];
        if (nw) x[(size_t)r * D + c] += dyt(v, alpha, nw[c], nb[c]);
        else x[(size_t)r * D + c] = v;                            // no norm given: the plain sum
    }
}

__global__ void dyt_gather_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ nw,
                                  const float* __restrict__ nb, float alpha, float* __restrict__ out,
                                  __nv_bfloat16* __restrict__ out_b, int D) {
    pdl_release();
    pdl_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float v = dyt(x[(size_t)r * D + c], alpha, nw[c], nb[c]);
        out[(size_t)blockIdx.x * D + c] = v;
        if (out_b) out_b[(size_t)blockIdx.x * D + c] = __float2bfloat16_rn(v);
    }
}

// greedy sampling: index of the largest logit of every row (ties: the lowest index)
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.x * V;
    float best = -CUDART_INF_F;
    int at = 0x7fffffff;
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
        const float v = row[c];
        if (v > best || (v == best && c < at)) { best = v; at = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > best || (ov == best && oi < at)) { best = ov; at = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = at; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (bv[w] > best || (bv[w] == best && bi[w] < at)) { best = bv[w]; at = bi[w]; }
        out[blockIdx.x] = at;
    }
}

// ---- launchers --------------------------------------------------------------------------------------------------------
cudaError_t launch_embed(const void* table, const int* ids, float* out, int M, int V, int D, cudaStream_t st) {
    return launch_pdl(embed_rows_bf16_kernel, dim3(M), dim3(128), 0, st, reinterpret_cast<const __nv_bfloat16*>(table), ids, out, V, D);
}

static inline int col_blocks(int D) { return D > 1024 ? (D + 1023) / 1024 : 1; }

cudaError_t launch_dyt_tapmix(const float* x, const NormW& n, const float* cw, int taps, const float* tail, const RowMeta& rm,
                              float* out, void* out_bf16, int M, int D, cudaStream_t st) {
    dyt_tapmix_kernel<<<dim3(M, col_blocks(D)), 256, 0, st>>>(x, n.w, n.b, n.alpha, cw, taps, tail, rm.slot, rm.pos, rm.start,
                                                              out, reinterpret_cast<__nv_bfloat16*>(out_bf16), D);
    return cudaGetLastError();
}

cudaError_t launch_tapmix_tail(const float* x, const NormW& n, int taps, float* tail, const SeqMeta& sm, int n_seq, int D,
                               cudaStream_t st) {
    if (taps <= 1) return cudaSuccess;
    tapmix_tail_kernel<<<dim3(n_seq, col_blocks(D)), 256, 0, st>>>(x, n.w, n.b, n.alpha, taps, tail, sm.slot, sm.row0, sm.count, D);
    return cudaGetLastError();
}

cudaError_t launch_linear(const float* A, int lda, const void* W, long long w_expert_stride, float* Y, int ldy, int M, int N,
                          int K, const GroupMap* gm, cudaStream_t st) {
    const int* a_row = gm ? gm->a_row : nullptr;
    const float* a_scale = gm ? gm->a_scale : nullptr;
    const int* a_expert = gm ? gm->a_expert : nullptr;
    const int* n_slots = gm ? gm->n_slots : nullptr;
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(W);
    // a few rows, or a few outputs (router logits: the same kernel for every step length, so that the choice of experts
    // does not depend on how a prompt was cut)
    if (M <= kRowsKernelMax || (N <= kRowsKernelMaxOut && M <= 65535))
        return launch_pdl(linear_rows_kernel, dim3((N + 7) / 8, M), dim3(256), 0, st, A, lda, w, w_expert_stride, Y, ldy, M, N, K,
                          a_row, a_scale, a_expert, n_slots, (float*)nullptr, (const float*)nullptr, (const float*)nullptr, 0.f,
                          TapOut{});
    else
        linear_tile_kernel<<<dim3((N + BN - 1) / BN, (M + BM - 1) / BM), 256, 0, st>>>(A, lda, w, w_expert_stride, Y, ldy, M, N,
                                                                                      K, a_row, a_scale, a_expert, n_slots);
    return cudaGetLastError();
}

// ---- the fused forms for a step of a few rows ----
cudaError_t launch_dyt_tapmix_seq(const float* x, const NormW& n, const float* cw, int taps, float* tail, const SeqMeta& sm,
                                  const RowMeta& rm, int n_seq, float* out, int D, cudaStream_t st) {
    return launch_pdl(dyt_tapmix_seq_kernel, dim3(n_seq, (D + 127) / 128), dim3(128), 0, st, x, n.w, n.b, n.alpha, cw, taps, tail,
                      sm.slot, sm.row0, sm.count, rm.pos, out, D);
}

cudaError_t launch_linear_rows_residual(const float* A, int lda, const void* W, float* x, int M, int N, int K, const NormW& n,
                                        const TapOut& next, cudaStream_t st) {
    return launch_pdl(linear_rows_kernel, dim3((N + 7) / 8, M), dim3(256), 0, st, A, lda, reinterpret_cast<const __nv_bfloat16*>(W),
                      0LL, (float*)nullptr, N, M, N, K, (const int*)nullptr, (const float*)nullptr, (const int*)nullptr,
                      (const int*)nullptr, x, n.w, n.b, n.alpha, next);
}

cudaError_t launch_gated_rows(const float* A, int lda, const void* W, long long w_expert_stride, float* mid, int n_assign, int F,
                              int K, const GroupMap* gm, const void* Ws, float* smid, int n_shared_rows, int Sf, cudaStream_t st,
                              const GluAct& act) {
    const int widest = std::max(F, n_shared_rows > 0 ? Sf : 0);
    return launch_pdl(gated_rows_kernel, dim3((widest + 7) / 8, n_assign + n_shared_rows), dim3(256), 0, st, A, lda,
                      reinterpret_cast<const __nv_bfloat16*>(W), w_expert_stride, mid, n_assign, F, K,
                      gm ? (const int*)gm->a_row : nullptr, gm ? (const float*)gm->a_scale : nullptr,
                      gm ? (const int*)gm->a_expert : nullptr, reinterpret_cast<const __nv_bfloat16*>(Ws), smid, Sf, act);
}

cudaError_t launch_down_combine_rows(const float* mid, int F, const void* Wd, const int* a_expert, int top, const float* smid,
                                     int Sf, const void* Wsd, float* x, int M, int D, const NormW& n, const TapOut& next,
                                     cudaStream_t st, const float* a_weight, int n_real, const float* ident_h,
                                     const float* shared_gate, int shared_gate_ld) {
    return launch_pdl(down_combine_rows_kernel, dim3((D + 7) / 8, M), dim3(256), 0, st, mid, F,
                      reinterpret_cast<const __nv_bfloat16*>(Wd), a_expert, top, smid, Sf, reinterpret_cast<const __nv_bfloat16*>(Wsd), x,
                      D, n.w, n.b, n.alpha, next, a_weight, n_real, ident_h, shared_gate, shared_gate_ld);
}

cudaError_t launch_router_rows(const float* h, int D, const void* Wr, int E, int top, int M, float* z, const GroupMap& gm,
                               int* slot_of, cudaStream_t st, const float* bias, bool softmax_top, const GroupedRoute* gr) {
    const GroupedRoute rule = gr ? *gr : GroupedRoute{};
    return launch_pdl(router_rows_kernel, dim3(M), dim3(256), (size_t)(E + rule.n + rule.count) * sizeof(float), st, h, D,
                      reinterpret_cast<const __nv_bfloat16*>(Wr), E, top, z, gm.a_row, gm.a_scale, gm.a_expert, slot_of, gm.n_slots,
                      bias, softmax_top ? 1 : 0, rule);
}

cudaError_t launch_qk_norm_cache(float* qk, int nq, int nk, const float* qw, const float* kw, float eps, float* kcache,
                                 float* vcache, const PageMap& pm, int kv_heads, int dim, const RowMeta& rm, int M,
                                 cudaStream_t st) {
    return launch_pdl(qk_norm_cache_kernel, dim3(M), dim3(256), 0, st, qk, nq, nk, qw, kw, eps, kcache, vcache, pm.table,
                      pm.max_pages, pm.page_size, kv_heads, dim, rm.slot, rm.pos);
}

template <int NC>
static cudaError_t launch_attention_tiles(const float* qk, int q_stride, const float* kcache, const float* vcache,
                                          const PageMap& pm, const AttnShape& a, const RowMeta& rm, float* out,
                                          __nv_bfloat16* out_b, int M, cudaStream_t st) {
    constexpr int DP = 64 * NC;
    const size_t smem = (size_t)(2 * kTQ * (DP + 4) + kTK * DP + kTQ * kTPStride) * sizeof(float) + 2 * kTQ * sizeof(int);
    static bool attr[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !attr[dev]) {
        e = cudaFuncSetAttribute(sink_attention_tile_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr[dev] = true;
    }
    sink_attention_tile_kernel<NC><<<dim3((M + kTQ - 1) / kTQ, a.heads), kTileThreads, smem, st>>>(
        qk, q_stride, kcache, vcache, pm.table, pm.max_pages, pm.page_size, a.heads, a.kv_heads, a.dim, a.scale, a.softcap,
        a.temp, a.slopes, a.sink, a.window, a.keep_first, rm.slot, rm.pos, out, out_b, M);
    return cudaGetLastError();
}

template <int HG>
static cudaError_t launch_attention_splits(const float* qk, int q_stride, const float* kcache, const float* vcache,
                                           const PageMap& pm, const AttnShape& a, const RowMeta& rm, float* out,
                                           __nv_bfloat16* out_b, int M, float* split_ws, unsigned* arrived, cudaStream_t st) {
    const int group = a.heads / a.kv_heads, chunks = (group + HG - 1) / HG;
    // enough CTAs for two per SM, at least 16 keys per split where the window bounds the keys
    const long long max_keys = a.window > 0 ? (long long)a.window + a.keep_first : (long long)pm.max_pages * pm.page_size;
    const int others = M * a.kv_heads * chunks;
    int S = (2 * 148 + others - 1) / others;
    S = (int)std::max<long long>(1, std::min<long long>(std::min(S, kAttnSplitsMax), (max_keys + 15) / 16));
    return launch_pdl(sink_attention_split_kernel<HG>, dim3(M, a.kv_heads * chunks, S), dim3(kSplitThreads), 0, st, qk, q_stride,
                      kcache, vcache, pm.table, pm.max_pages, pm.page_size, a.heads, a.kv_heads, a.dim, a.scale, a.softcap, a.temp,
                      a.slopes, a.sink, a.window, a.keep_first, rm.slot, rm.pos, split_ws, arrived, out, out_b);
}

// a step of a few rows (decoding) splits every row's keys over CTAs; longer steps run the tiled kernel.
// split_ws: kRowsKernelMax * heads * kAttnSplitsMax * (dim + 2) floats; arrived: kRowsKernelMax * heads zeroed counters
cudaError_t launch_sink_attention(const float* qk, int q_stride, const float* kcache, const float* vcache, const PageMap& pm,
                                  const AttnShape& a, const RowMeta& rm, float* out, void* out_bf16, float* split_ws,
                                  unsigned* arrived, int M, cudaStream_t st) {
    if (a.dim > 32 * kAttnMaxDimPerLane || a.heads % a.kv_heads) return cudaErrorNotSupported;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(out_bf16);
    if (M > kAttnRowsKernelMax) {
        switch ((a.dim + 63) / 64) {
            case 1: return launch_attention_tiles<1>(qk, q_stride, kcache, vcache, pm, a, rm, out, ob, M, st);
            case 2: return launch_attention_tiles<2>(qk, q_stride, kcache, vcache, pm, a, rm, out, ob, M, st);
            case 3: return launch_attention_tiles<3>(qk, q_stride, kcache, vcache, pm, a, rm, out, ob, M, st);
            default: return launch_attention_tiles<4>(qk, q_stride, kcache, vcache, pm, a, rm, out, ob, M, st);
        }
    }
    const int group = a.heads / a.kv_heads;
    if (group >= 4) return launch_attention_splits<4>(qk, q_stride, kcache, vcache, pm, a, rm, out, ob, M, split_ws, arrived, st);
    if (group >= 2) return launch_attention_splits<2>(qk, q_stride, kcache, vcache, pm, a, rm, out, ob, M, split_ws, arrived, st);
    return launch_attention_splits<1>(qk, q_stride, kcache, vcache, pm, a, rm, out, ob, M, split_ws, arrived, st);
}

cudaError_t launch_router_topk(const float* z, int E, int top, int M, int* sel_e, float* sel_w, cudaStream_t st, const float* bias,
                               bool softmax_top, const GroupedRoute* gr) {
    const GroupedRoute rule = gr ? *gr : GroupedRoute{};
    router_topk_kernel<<<(M + 3) / 4, 128, (size_t)4 * (rule.n + rule.count) * sizeof(float), st>>>(z, E, top, M, sel_e, sel_w, bias,
                                                                                                    softmax_top ? 1 : 0, rule);
    return cudaGetLastError();
}

cudaError_t launch_moe_group(const int* sel_e, const float* sel_w, int n_assign, int top, int E, int pad, const GroupMap& gm,
                             int* slot_of, int max_slots, cudaStream_t st) {
    moe_group_kernel<<<1, 256, 3 * E * sizeof(int), st>>>(sel_e, sel_w, n_assign, top, E, pad, gm.a_row, gm.a_scale, gm.a_expert,
                                                          slot_of, gm.n_slots, max_slots);
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(const float* gu, float* mid, void* mid_bf16, int M, int F, const GroupMap* gm, cudaStream_t st, int act,
                            float limit) {
    silu_mul_kernel<<<M, 256, 0, st>>>(gu, mid, reinterpret_cast<__nv_bfloat16*>(mid_bf16), F, gm ? gm->a_row : nullptr,
                                       gm ? gm->n_slots : nullptr, M, act, limit);
    return cudaGetLastError();
}

cudaError_t launch_pack_rows_bf16(const float* A, void* Ab, int M, int D, const GroupMap* gm, cudaStream_t st) {
    pack_rows_bf16_kernel<<<M, 256, 0, st>>>(A, reinterpret_cast<__nv_bfloat16*>(Ab), D, gm ? gm->a_row : nullptr,
                                             gm ? gm->a_scale : nullptr, gm ? gm->n_slots : nullptr, M);
    return cudaGetLastError();
}

cudaError_t launch_residual_dyt(float* x, const float* y, const float* parts, const int* slot_of, int top, const NormW& n, int M,
                                int D, cudaStream_t st) {
    residual_dyt_kernel<<<dim3(M, col_blocks(D)), 256, 0, st>>>(x, y, parts, slot_of, top, n.w, n.b, n.alpha, D);
    return cudaGetLastError();
}

cudaError_t launch_dyt_gather(const float* x, const int* rows, const NormW& n, float* out, void* out_bf16, int M, int D,
                              cudaStream_t st) {
    return launch_pdl(dyt_gather_kernel, dim3(M), dim3(256), 0, st, x, rows, n.w, n.b, n.alpha, out,
                      reinterpret_cast<__nv_bfloat16*>(out_bf16), D);
}

cudaError_t launch_argmax_rows(const float* logits, int M, int V, int* out, cudaStream_t st) {
    argmax_rows_kernel<<<M, 256, 0, st>>>(logits, V, out);
    return cudaGetLastError();
}

}  // namespace lm

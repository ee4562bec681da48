// Fused GAT forward / backward for sm_100a.
//
// Forward: one sweep over each destination row.  A warp owns the row's H*F
// output floats as float4 vectors (lane l holds vectors l, l+32, ...), reads 32
// column ids at a time with one coalesced load, then gathers the source rows
// four edges at a time (each gather is a contiguous H*F*4-byte row, 16 B per
// lane) while an online softmax keeps (max, sum, weighted accumulator) per head
// in registers -- column ids and attention terms are read once, features once.
// Rows longer than DGNN_SEG edges are split (see common.cuh); no atomics.
//
// Backward: S[r,h] = <grad_out[r,h,:], out[r,h,:]> replaces the reference's
// per-row edge sweep, so one pass over the CSC form yields grad_feat,
// grad_attn_col and the per-edge term d_e (scattered to CSR order), and a
// streaming row reduction of d_e yields grad_attn_row.  Two feature gathers in
// total for forward+backward instead of three, and no float atomics.
#include "common.cuh"
#include "gat_sh.cuh"

namespace {

template <int VPL> struct Unroll { static constexpr int U = VPL <= 2 ? 4 : 2; };

// ------------------------------------------------------------------ forward
template <int VPL, bool MASK, bool FULL, int LPR, bool NEG>
struct GatFwdOp {
  static constexpr int EPW = 32 / LPR;
  static constexpr int MIN_BLOCKS = VPL <= 2 ? 5 : (VPL == 4 ? 4 : 2);
  static constexpr bool HAS_PARTIALS = true;
  i64 n_rows, nnz;
  const void* indptr;
  int idx_bits;
  int H, hf4, f4_shift;
  const int* col_ind;
  const float* attn_row;
  const float* attn_col;
  const float4* in_feat;
  const float* mask;
  float slope, drop_p, inv_keep;
  float4* out;
  float* edge_max;
  float* edge_sum;
  float* ws;
  i64 slot_stride;  // floats per partial slot
  // staged sweep over column blocks: the (max, sum, accumulator) state of every row is
  // carried in `state` (one slot per row) between calls; first / last mark the ends
  float* state;
  int first, last, skip_empty;
  static constexpr bool STAGED = true;
  const unsigned char* stage_mask;   // per row: bit p set = the row has entries in stage p (NULL: every row in every stage)
  int stage;
  const unsigned* hot;   // accepted for symmetry with the same-head operators; this layout loads every row plainly
  const float4* bias;   // optional [H*F] added to the normalised output (layer epilogue)
  // NEG: the share of the result that comes from edges on the negative side of the LeakyReLU
  float4* out_neg;      // [n_rows, H*F], normalised like out (no bias)
  float* a_neg;         // [n_rows, H]: sum of alpha over those edges

  struct State {
    LaneMap<VPL, LPR> lm;
    float ar[VPL], m[VPL], z[VPL], zn[NEG ? VPL : 1];
    float4 acc[VPL];
    float4 accn[NEG ? VPL : 1];
  };

  __device__ __forceinline__ void init(State& st, i64 r, int lane) const {
    st.lm.init(lane, hf4, f4_shift);
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      st.ar[v] = st.lm.act[v] ? __ldg(attn_row + r * H + st.lm.hd[v]) : 0.f;
      st.m[v] = DGNN_NEG_INIT;
      st.z[v] = 0.f;
      st.acc[v] = zero4();
      if (NEG) { st.zn[v] = 0.f; st.accn[v] = zero4(); }
    }
  }
  __device__ __forceinline__ void resume(State& st, i64 r, int lane, bool first_) const {
    if (!first_ && st.lm.sg == 0) merge_partial(st, state + r * slot_stride, lane);
  }
  // fold the (max, sum, accumulator) of the sub-groups; afterwards every sub-group holds the row's state
  __device__ __forceinline__ void combine(State& st, int) const {
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) {
      const float mo = __shfl_xor_sync(DGNN_FULL, st.m[0], off);
      const float zo = __shfl_xor_sync(DGNN_FULL, st.z[0], off);
      float4 ao;
      ao.x = __shfl_xor_sync(DGNN_FULL, st.acc[0].x, off);
      ao.y = __shfl_xor_sync(DGNN_FULL, st.acc[0].y, off);
      ao.z = __shfl_xor_sync(DGNN_FULL, st.acc[0].z, off);
      ao.w = __shfl_xor_sync(DGNN_FULL, st.acc[0].w, off);
      const float mn = fmaxf(st.m[0], mo);
      const float s1 = fast_exp(st.m[0] - mn), s2 = fast_exp(mo - mn);
      // both partners must compute the same sum: add in a fixed (lower sub-group first) order
      const bool low = (st.lm.sg & (off / LPR)) == 0;
      const float za = low ? st.z[0] * s1 : zo * s2, zb = low ? zo * s2 : st.z[0] * s1;
      st.z[0] = za + zb;
      float4 a = st.acc[0], b = ao;
      scale4(a, s1);
      scale4(b, s2);
      if (!low) { const float4 t = a; a = b; b = t; }
      add4(a, b);
      st.acc[0] = a;
      if (NEG) {
        const float no = __shfl_xor_sync(DGNN_FULL, st.zn[0], off);
        float4 co;
        co.x = __shfl_xor_sync(DGNN_FULL, st.accn[0].x, off);
        co.y = __shfl_xor_sync(DGNN_FULL, st.accn[0].y, off);
        co.z = __shfl_xor_sync(DGNN_FULL, st.accn[0].z, off);
        co.w = __shfl_xor_sync(DGNN_FULL, st.accn[0].w, off);
        const float na = low ? st.zn[0] * s1 : no * s2, nb = low ? no * s2 : st.zn[0] * s1;
        st.zn[0] = na + nb;
        float4 c = st.accn[0], d = co;
        scale4(c, s1);
        scale4(d, s2);
        if (!low) { const float4 t = c; c = d; d = t; }
        add4(c, d);
        st.accn[0] = c;
      }
      st.m[0] = mn;
    }
  }

  // one batch of U edges per sub-group starting at tile slot k; ALL = every slot of the batch holds an edge
  template <bool ALL>
  __device__ __forceinline__ void batch(State& st, int my_c, i64 ebase, int k, int cnt) const {
    constexpr int U = Unroll<VPL>::U;
    int c[U], slot[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      slot[u] = k + u * EPW + st.lm.sg;      // tile slot of this sub-group's u-th edge
      c[u] = __shfl_sync(DGNN_FULL, my_c, slot[u] & 31);
    }
    float s[U][VPL];
    float4 x[U][VPL];
    bool keep[U][VPL];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const bool ok = (ALL || slot[u] < cnt) && (FULL || st.lm.act[v]);
        s[u][v] = ok ? __ldg(attn_col + (i64)c[u] * H + st.lm.hd[v]) : 0.f;
        x[u][v] = ok ? ld4(in_feat + (i64)c[u] * hf4 + st.lm.q[v]) : zero4();
        keep[u][v] = ok;
        if (MASK) keep[u][v] = ok ? (__ldg(mask + (ebase + slot[u]) * H + st.lm.hd[v]) > drop_p) : false;
      }
    }
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      float l[U];
      float bm = st.m[v];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        l[u] = (ALL || slot[u] < cnt) ? leaky(st.ar[v] + s[u][v], slope) : DGNN_NEG_INIT;
        bm = fmaxf(bm, l[u]);
      }
      // rescale only when the running maximum moved for some lane of the warp
      const bool moved = __any_sync(DGNN_FULL, bm > st.m[v]);
      if (!FULL && !st.lm.act[v]) { st.m[v] = bm; continue; }
      if (moved) {
        const float sc = fast_exp(st.m[v] - bm);
        st.z[v] *= sc;
        scale4(st.acc[v], sc);
        if (NEG) { st.zn[v] *= sc; scale4(st.accn[v], sc); }
        st.m[v] = bm;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (ALL || slot[u] < cnt) {
          const float p = fast_exp(l[u] - bm);
          st.z[v] += p;
          const float pn = l[u] < 0.f ? p : 0.f;
          if (NEG) st.zn[v] += pn;
          if (!MASK || keep[u][v]) {
            fma4(st.acc[v], p, x[u][v]);
            if (NEG) fma4(st.accn[v], pn, x[u][v]);
          }
        }
      }
    }
  }

  __host__ __device__ __forceinline__ int ring_bytes() const { return 0; }   // gathers go straight into registers
  __device__ __forceinline__ void range(State& st, i64, i64 e0, i64 e1, int lane, float4*) const {
    constexpr int STEP = Unroll<VPL>::U * EPW;
    for (i64 base = e0; base < e1; base += 32) {
      const int cnt = (int)((e1 - base) < 32 ? (e1 - base) : 32);
      const int my_c = lane < cnt ? __ldg(col_ind + base + lane) : 0;
      int k = 0;
      for (; k + STEP <= cnt; k += STEP) batch<true>(st, my_c, base, k, cnt);
      if (k < cnt) batch<false>(st, my_c, base, k, cnt);
    }
  }

  __device__ __forceinline__ void finalize(State& st, i64 r, int lane, bool last_) const {
    if (!last_) { store_partial(st, state + r * slot_stride, lane); return; }
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (!st.lm.act[v]) continue;
      if (!st.lm.wr[v]) continue;
      const float sc = st.z[v] > 0.f ? inv_keep / st.z[v] : 0.f;
      float4 a = st.acc[v];
      scale4(a, sc);
      if (bias) add4(a, __ldg(bias + st.lm.q[v]));
      out[r * hf4 + st.lm.q[v]] = a;
      if (NEG) {
        float4 an = st.accn[v];
        scale4(an, sc);
        out_neg[r * hf4 + st.lm.q[v]] = an;
      }
      if (st.lm.wlead[v] && edge_max) {
        edge_max[r * H + st.lm.hd[v]] = st.m[v];
        edge_sum[r * H + st.lm.hd[v]] = st.z[v];
      }
      if (NEG && st.lm.wlead[v]) a_neg[r * H + st.lm.hd[v]] = st.z[v] > 0.f ? st.zn[v] / st.z[v] : 0.f;
    }
  }

  // slot layout: [acc H*F | m H | z H | (NEG: zn H) | pad to 4 | (NEG: accn H*F)]
  __device__ __forceinline__ void store_partial(State& st, float* p, int) const {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (!st.lm.wr[v]) continue;
      reinterpret_cast<float4*>(p)[st.lm.q[v]] = st.acc[v];
      if (NEG) reinterpret_cast<float4*>(p + slot_stride - hf4 * 4)[st.lm.q[v]] = st.accn[v];
      if (st.lm.wlead[v]) {
        p[hf4 * 4 + st.lm.hd[v]] = st.m[v];
        p[hf4 * 4 + H + st.lm.hd[v]] = st.z[v];
        if (NEG) p[hf4 * 4 + 2 * H + st.lm.hd[v]] = st.zn[v];
      }
    }
  }

  __device__ __forceinline__ void merge_partial(State& st, const float* p, int) const {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (!st.lm.act[v]) continue;
      const float4 ai = reinterpret_cast<const float4*>(p)[st.lm.q[v]];
      const float mi = p[hf4 * 4 + st.lm.hd[v]];
      const float zi = p[hf4 * 4 + H + st.lm.hd[v]];
      const float mn = fmaxf(st.m[v], mi);
      const float s1 = fast_exp(st.m[v] - mn), s2 = fast_exp(mi - mn);
      st.z[v] = st.z[v] * s1 + zi * s2;
      scale4(st.acc[v], s1);
      fma4(st.acc[v], s2, ai);
      if (NEG) {
        st.zn[v] = st.zn[v] * s1 + p[hf4 * 4 + 2 * H + st.lm.hd[v]] * s2;
        scale4(st.accn[v], s1);
        fma4(st.accn[v], s2, reinterpret_cast<const float4*>(p + slot_stride - hf4 * 4)[st.lm.q[v]]);
      }
      st.m[v] = mn;
    }
  }
};

// any H, F: one warp per (row, head), lanes over features (slow path)
__global__ void __launch_bounds__(DGNN_THREADS)
k_gat_fwd_generic(i64 n_rows, int H, int F, const void* indptr, int idx_bits, const int* col_ind,
                  const float* attn_row, const float* attn_col, const float* in_feat,
                  const float* mask, float slope, float drop_p, float inv_keep,
                  float* out, float* edge_max, float* edge_sum) {
  const int lane = threadIdx.x & 31;
  const i64 w = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  if (w >= n_rows * H) return;
  const i64 r = w / H;
  const int h = (int)(w % H);
  const i64 lb = ldp(indptr, idx_bits, r), hb = ldp(indptr, idx_bits, r + 1);
  const float ar = __ldg(attn_row + r * H + h);
  float m = DGNN_NEG_INIT;
  for (i64 e = lb + lane; e < hb; e += 32)
    m = fmaxf(m, leaky(ar + __ldg(attn_col + (i64)col_ind[e] * H + h), slope));
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(DGNN_FULL, m, o));
  float z = 0.f;
  for (i64 e = lb + lane; e < hb; e += 32)
    z += expf(leaky(ar + __ldg(attn_col + (i64)col_ind[e] * H + h), slope) - m);
  for (int o = 16; o; o >>= 1) z += __shfl_xor_sync(DGNN_FULL, z, o);
  if (lane == 0 && edge_max) { edge_max[r * H + h] = m; edge_sum[r * H + h] = z; }
  const float sc = z > 0.f ? inv_keep / z : 0.f;
  for (int fb = lane; fb < F; fb += 32) {
    float acc = 0.f;
    for (i64 e = lb; e < hb; ++e) {
      const i64 c = col_ind[e];
      if (mask && !(__ldg(mask + e * H + h) > drop_p)) continue;
      const float p = expf(leaky(ar + __ldg(attn_col + c * H + h), slope) - m);
      acc = fmaf(p, __ldg(in_feat + (c * H + h) * F + fb), acc);
    }
    out[(r * H + h) * F + fb] = acc * sc;
  }
}

// ------------------------------------------------------------------ rowstat
template <int VPL>
__global__ void __launch_bounds__(DGNN_THREADS)
k_gat_rowstat(i64 n_rows, int H, int hf4, int f4_shift, const float* attn_row, const float* edge_max,
              const float* edge_sum, const float4* out, const float4* grad, float4* pack) {
  const int lane = threadIdx.x & 31;
  const i64 r = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  LaneMap<VPL> lm;
  lm.init(lane, hf4, f4_shift);
  float s[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v)
    s[v] = lm.act[v] ? dot4(ld4(grad + r * hf4 + lm.q[v]), ld4(out + r * hf4 + lm.q[v])) : 0.f;
  head_reduce<VPL>(s, f4_shift);
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    if (lm.lead[v]) {
      const i64 i = r * H + lm.hd[v];
      pack[i] = make_float4(__ldg(attn_row + i), __ldg(edge_max + i), 1.f / __ldg(edge_sum + i), s[v]);
    }
  }
}

// The same statistics in one pass with everything the layer's backward needs from the destination rows:
//  * bias != NULL: the forward added it to `out`, so the row term uses out - bias, and the bias gradient
//    sum_r grad[r,:] is accumulated on the way (a lane owns the same columns in every row; fixed-order
//    fold per CTA into part[cta][hf4], then over CTAs by k_bias_grad_final);
//  * out_neg != NULL: grad_attn_row[r,h] = (1 - slope) * (S * a_neg - <grad, out_neg>), which equals the
//    sum over the row's edges of alpha (g - S) (slope where the LeakyReLU is on its negative side) of the
//    reference (fused_backward_kernel, fused_gatconv_kernel.cu:931-957) with no per-edge array;
//  * grad_copy != NULL: grad is also written there (the buffer that the other ranks read on the sharded path).
//  * fan.ptr != NULL: row r's grad and pack are also written to the send-buffer rows fan.pos[fan.ptr[r]..fan.ptr[r+1])
//    (one per peer and chunk of the sharded layer that fetches the row), so no separate packing pass is needed.
struct RowFan {
  const int* ptr;
  const int* pos;
  float4* grad;   // [send rows, hf4]
  float4* pack;   // [send rows, H]
};

template <int VPL>
__global__ void __launch_bounds__(DGNN_THREADS)
k_gat_rowstat_full(i64 n_rows, int H, int hf4, int f4_shift, const float* attn_row, const float* edge_max,
                   const float* edge_sum, const float4* out, const float4* grad, const float4* bias,
                   const float4* out_neg, const float* a_neg, float one_minus_slope,
                   float4* pack, float* grad_attn_row, float4* grad_copy, float4* part, const RowFan fan) {
  extern __shared__ float4 rs_sm[];   // [DGNN_WARPS][hf4]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  LaneMap<VPL> lm;
  lm.init(lane, hf4, f4_shift);
  float4 b4[VPL], gsum[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    b4[v] = (bias && lm.act[v]) ? ld4(bias + lm.q[v]) : zero4();
    gsum[v] = zero4();
  }
  // two rows per warp and step: all their loads are issued before the first reduction
  constexpr int RS_ROWS = 2;
  const i64 stride = (i64)gridDim.x * DGNN_WARPS;
  for (i64 r0 = (i64)blockIdx.x * DGNN_WARPS + warp; r0 < n_rows; r0 += stride * RS_ROWS) {
    float4 g[RS_ROWS][VPL], o[RS_ROWS][VPL], on[RS_ROWS][VPL];
    float4 sc[RS_ROWS][VPL];   // per head (lead lanes): attn_row, edge_max, edge_sum, a_neg -- requested with the rows
#pragma unroll
    for (int k = 0; k < RS_ROWS; ++k) {
      const i64 r = r0 + k * stride;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const bool ok = lm.act[v] && r < n_rows;
        g[k][v] = ok ? ld4(grad + r * hf4 + lm.q[v]) : zero4();
        o[k][v] = ok ? ld4(out + r * hf4 + lm.q[v]) : zero4();
        on[k][v] = (ok && out_neg) ? ld4(out_neg + r * hf4 + lm.q[v]) : zero4();
        sc[k][v] = zero4();
        if (lm.lead[v] && r < n_rows) {
          const i64 i = r * H + lm.hd[v];
          sc[k][v] = make_float4(__ldg(attn_row + i), __ldg(edge_max + i), __ldg(edge_sum + i), out_neg ? __ldg(a_neg + i) : 0.f);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < RS_ROWS; ++k) {
      const i64 r = r0 + k * stride;
      if (r >= n_rows) break;            // uniform per warp
      float s[VPL], t[VPL];
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        s[v] = 0.f;
        t[v] = 0.f;
        if (lm.act[v]) {
          float4 ob = o[k][v];
          ob.x -= b4[v].x; ob.y -= b4[v].y; ob.z -= b4[v].z; ob.w -= b4[v].w;
          s[v] = dot4(g[k][v], ob);
          if (out_neg) t[v] = dot4(g[k][v], on[k][v]);
          if (grad_copy) grad_copy[r * hf4 + lm.q[v]] = g[k][v];
          add4(gsum[v], g[k][v]);
        }
      }
      head_reduce<VPL>(s, f4_shift);
      if (out_neg) head_reduce<VPL>(t, f4_shift);
      float4 pk[VPL];
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        pk[v] = zero4();
        if (lm.lead[v]) {
          const i64 i = r * H + lm.hd[v];
          pk[v] = make_float4(sc[k][v].x, sc[k][v].y, 1.f / sc[k][v].z, s[v]);
          pack[i] = pk[v];
          if (out_neg) grad_attn_row[i] = one_minus_slope * (s[v] * sc[k][v].w - t[v]);
        }
      }
      if (fan.ptr) {
        const int lo = __ldg(fan.ptr + r), hi = __ldg(fan.ptr + r + 1);
        for (int j = lo; j < hi; ++j) {
          const i64 p = __ldg(fan.pos + j);
#pragma unroll
          for (int v = 0; v < VPL; ++v) {
            if (!lm.act[v]) continue;
            fan.grad[p * hf4 + lm.q[v]] = g[k][v];
            if (lm.lead[v]) fan.pack[p * H + lm.hd[v]] = pk[v];
          }
        }
      }
    }
  }
  if (!part) return;
#pragma unroll
  for (int v = 0; v < VPL; ++v)
    if (lm.act[v]) rs_sm[warp * hf4 + lm.q[v]] = gsum[v];
  __syncthreads();
  for (int i = threadIdx.x; i < hf4; i += DGNN_THREADS) {
    float4 t4 = zero4();
    for (int w = 0; w < DGNN_WARPS; ++w) add4(t4, rs_sm[w * hf4 + i]);
    part[(i64)blockIdx.x * hf4 + i] = t4;
  }
}

__global__ void k_bias_grad_final(int ctas, int hf4, const float4* part, float4* grad_bias) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= hf4) return;
  float4 t = zero4();
  for (int c = 0; c < ctas; ++c) add4(t, part[(i64)c * hf4 + i]);
  grad_bias[i] = t;
}

__global__ void __launch_bounds__(DGNN_THREADS)
k_gat_rowstat_generic(i64 n_rows, int H, int F, const float* attn_row, const float* edge_max,
                      const float* edge_sum, const float* out, const float* grad, float4* pack) {
  const int lane = threadIdx.x & 31;
  const i64 w = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  if (w >= n_rows * H) return;
  float s = 0.f;
  for (int f = lane; f < F; f += 32) s = fmaf(__ldg(grad + w * F + f), __ldg(out + w * F + f), s);
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(DGNN_FULL, s, o);
  if (lane == 0) pack[w] = make_float4(attn_row[w], edge_max[w], 1.f / edge_sum[w], s);
}

// ------------------------------------------------------------ backward cols
template <int VPL, bool MASK, bool FULL, int LPR>
struct GatBwdOp {
  static constexpr int EPW = 32 / LPR;
  static constexpr int MIN_BLOCKS = VPL <= 2 ? 4 : (VPL == 4 ? 3 : 2);
  static constexpr bool HAS_PARTIALS = true;
  i64 n_rows, nnz;      // "rows" of the CSC form = source columns
  const void* indptr;   // col_ptr
  int idx_bits;
  int H, hf4, f4_shift;
  const int* row_ind;
  const int* permute;
  const float4* pack;
  const float* mask;
  const float4* in_feat;
  const float* attn_col;
  const float4* grad_out;
  float slope, drop_p, inv_keep;
  float4* grad_feat;
  float* grad_attn_col;
  float* grad_edge;  // [nnz,H] in CSR order
  float* ws;
  i64 slot_stride;
  float* state;      // staged sweep over row blocks: (grad_feat, grad_attn_col) accumulators per column
  int first, last, skip_empty;
  static constexpr bool STAGED = true;
  const unsigned char* stage_mask;   // per row: bit p set = the row has entries in stage p (NULL: every row in every stage)
  int stage;
  const unsigned* hot;   // accepted for symmetry with the same-head operators; this layout loads every row plainly

  struct State {
    LaneMap<VPL, LPR> lm;
    float4 x[VPL], acc[VPL];
    float ac[VPL], gc[VPL];
  };

  __device__ __forceinline__ void init(State& st, i64 c, int lane) const {
    st.lm.init(lane, hf4, f4_shift);
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      st.x[v] = st.lm.act[v] ? ld4(in_feat + c * hf4 + st.lm.q[v]) : zero4();
      st.ac[v] = st.lm.act[v] ? __ldg(attn_col + c * H + st.lm.hd[v]) : 0.f;
      st.acc[v] = zero4();
      st.gc[v] = 0.f;
    }
  }
  __device__ __forceinline__ void resume(State& st, i64 c, int lane, bool first_) const {
    if (!first_ && st.lm.sg == 0) merge_partial(st, state + c * slot_stride, lane);
  }
  // sum the sub-groups' accumulators (lower sub-group first, so all partners agree bit for bit)
  __device__ __forceinline__ void combine(State& st, int) const {
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) {
      float4 ao;
      ao.x = __shfl_xor_sync(DGNN_FULL, st.acc[0].x, off);
      ao.y = __shfl_xor_sync(DGNN_FULL, st.acc[0].y, off);
      ao.z = __shfl_xor_sync(DGNN_FULL, st.acc[0].z, off);
      ao.w = __shfl_xor_sync(DGNN_FULL, st.acc[0].w, off);
      const float go = __shfl_xor_sync(DGNN_FULL, st.gc[0], off);
      const bool low = (st.lm.sg & (off / LPR)) == 0;
      float4 a = low ? st.acc[0] : ao, b = low ? ao : st.acc[0];
      add4(a, b);
      st.acc[0] = a;
      st.gc[0] = low ? st.gc[0] + go : go + st.gc[0];
    }
  }

  template <bool ALL>
  __device__ __forceinline__ void batch(State& st, int my_r, int my_p, int k, int cnt) const {
    constexpr int U = Unroll<VPL>::U;
    int r[U], pp[U], slot[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      slot[u] = k + u * EPW + st.lm.sg;      // tile slot of this sub-group's u-th edge
      r[u] = __shfl_sync(DGNN_FULL, my_r, slot[u] & 31);
      pp[u] = __shfl_sync(DGNN_FULL, my_p, slot[u] & 31);
    }
    float4 pk[U][VPL], g4[U][VPL];
    bool keep[U][VPL];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const bool ok = (ALL || slot[u] < cnt) && (FULL || st.lm.act[v]);
        pk[u][v] = ok ? ld4(pack + (i64)r[u] * H + st.lm.hd[v]) : zero4();
        g4[u][v] = ok ? ld4(grad_out + (i64)r[u] * hf4 + st.lm.q[v]) : zero4();
        keep[u][v] = ok;
        if (MASK) keep[u][v] = ok ? (__ldg(mask + (i64)pp[u] * H + st.lm.hd[v]) > drop_p) : false;
      }
    }
    float d[U][VPL];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int v = 0; v < VPL; ++v) d[u][v] = dot4(g4[u][v], st.x[v]);
    head_reduce<U, VPL>(d, f4_shift);  // executed by all lanes, also for slots past cnt
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ALL || slot[u] < cnt) {
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          if (!FULL && !st.lm.act[v]) continue;
          const float l = leaky(pk[u][v].x + st.ac[v], slope);
          const float alpha = fast_exp(l - pk[u][v].y) * pk[u][v].z;   // pack.z = 1 / edge_sum
          const float kp = (!MASK || keep[u][v]) ? inv_keep : 0.f;
          float de = alpha * (d[u][v] * kp - pk[u][v].w);
          de = l < 0.f ? de * slope : de;
          st.gc[v] += de;
          fma4(st.acc[v], alpha * kp, g4[u][v]);
          if (grad_edge && st.lm.lead[v]) grad_edge[(i64)pp[u] * H + st.lm.hd[v]] = de;
        }
      }
    }
  }

  __host__ __device__ __forceinline__ int ring_bytes() const { return 0; }   // gathers go straight into registers
  __device__ __forceinline__ void range(State& st, i64, i64 e0, i64 e1, int lane, float4*) const {
    constexpr int STEP = Unroll<VPL>::U * EPW;
    for (i64 base = e0; base < e1; base += 32) {
      const int cnt = (int)((e1 - base) < 32 ? (e1 - base) : 32);
      const int my_r = lane < cnt ? __ldg(row_ind + base + lane) : 0;
      // without a permutation the mask (if any) is laid out in CSC order: the position is the index
      const int my_p = lane < cnt ? (permute ? __ldg(permute + base + lane) : (int)(base + lane)) : 0;
      int k = 0;
      for (; k + STEP <= cnt; k += STEP) batch<true>(st, my_r, my_p, k, cnt);
      if (k < cnt) batch<false>(st, my_r, my_p, k, cnt);
    }
  }

  __device__ __forceinline__ void finalize(State& st, i64 c, int lane, bool last_) const {
    if (!last_) { store_partial(st, state + c * slot_stride, lane); return; }
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (!st.lm.wr[v]) continue;
      grad_feat[c * hf4 + st.lm.q[v]] = st.acc[v];
      if (st.lm.wlead[v]) grad_attn_col[c * H + st.lm.hd[v]] = st.gc[v];
    }
  }

  __device__ __forceinline__ void store_partial(State& st, float* p, int) const {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (!st.lm.wr[v]) continue;
      reinterpret_cast<float4*>(p)[st.lm.q[v]] = st.acc[v];
      if (st.lm.wlead[v]) p[hf4 * 4 + st.lm.hd[v]] = st.gc[v];
    }
  }

  __device__ __forceinline__ void merge_partial(State& st, const float* p, int) const {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (!st.lm.act[v]) continue;
      add4(st.acc[v], reinterpret_cast<const float4*>(p)[st.lm.q[v]]);
      st.gc[v] += p[hf4 * 4 + st.lm.hd[v]];
    }
  }
};

// any H, F: one warp per (column, head)
__global__ void __launch_bounds__(DGNN_THREADS)
k_gat_bwd_cols_generic(i64 n_cols, int H, int F, const void* col_ptr, int idx_bits, const int* row_ind,
                       const int* permute, const float4* pack, const float* mask, const float* in_feat,
                       const float* attn_col, const float* grad_out, float slope, float drop_p,
                       float inv_keep, float* grad_feat, float* grad_attn_col, float* grad_edge) {
  const int lane = threadIdx.x & 31;
  const i64 w = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  if (w >= n_cols * H) return;
  const i64 c = w / H;
  const int h = (int)(w % H);
  const i64 lb = ldp(col_ptr, idx_bits, c), hb = ldp(col_ptr, idx_bits, c + 1);
  const float ac = __ldg(attn_col + c * H + h);
  float gc = 0.f;
  for (i64 e = lb; e < hb; ++e) {
    const i64 r = row_ind[e];
    const i64 pp = permute ? (i64)permute[e] : e;
    const float4 pk = pack[r * H + h];
    float d = 0.f;
    for (int f = lane; f < F; f += 32)
      d = fmaf(__ldg(grad_out + (r * H + h) * F + f), __ldg(in_feat + (c * H + h) * F + f), d);
    for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(DGNN_FULL, d, o);
    const float l = leaky(pk.x + ac, slope);
    const float alpha = expf(l - pk.y) * pk.z;
    const float kp = (!mask || __ldg(mask + pp * H + h) > drop_p) ? inv_keep : 0.f;
    float de = alpha * (d * kp - pk.w);
    if (l < 0.f) de *= slope;
    gc += de;
    if (lane == 0 && grad_edge) grad_edge[pp * H + h] = de;
  }
  if (lane == 0) grad_attn_col[c * H + h] = gc;
  for (int fb = lane; fb < F; fb += 32) {
    float acc = 0.f;
    for (i64 e = lb; e < hb; ++e) {
      const i64 r = row_ind[e];
      const float4 pk = pack[r * H + h];
      const float kp = (!mask || __ldg(mask + (permute ? (i64)permute[e] : e) * H + h) > drop_p) ? inv_keep : 0.f;
      const float alpha = expf(leaky(pk.x + ac, slope) - pk.y) * pk.z;
      acc = fmaf(alpha * kp, __ldg(grad_out + (r * H + h) * F + fb), acc);
    }
    grad_feat[(c * H + h) * F + fb] = acc;
  }
}

// ------------------------------------------- row reduction of d_e (CSR order)
// one thread per (row, head); long rows go through chunk partials like the
// feature kernels so that every sum has a fixed order
__global__ void k_rowred_rows(i64 n_rows, int H, const void* indptr, int idx_bits,
                              const float* grad_edge, float* grad_attn_row, int all_rows) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_rows * H) return;
  const i64 r = t / H;
  const int h = (int)(t % H);
  const i64 lb = ldp(indptr, idx_bits, r), hb = ldp(indptr, idx_bits, r + 1);
  if (hb - lb > DGNN_SEG && !all_rows) return;
  float s = 0.f;
  for (i64 e = lb; e < hb; ++e) s += __ldg(grad_edge + e * H + h);
  grad_attn_row[t] = s;
}

__global__ void k_rowred_chunks(i64 n_rows, i64 nnz, int H, const void* indptr, int idx_bits,
                                const float* grad_edge, float* part) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  const i64 w = t / H;
  const int h = (int)(t % H);
  const i64 j = w >> 1;
  const int slot = (int)(w & 1);
  const i64 cs = j * DGNN_SEG;
  if (cs >= nnz) return;
  const i64 ce = (cs + DGNN_SEG < nnz) ? cs + DGNN_SEG : nnz;
  const i64 r = find_row(indptr, idx_bits, n_rows, slot ? ce - 1 : cs);
  const i64 lb = ldp(indptr, idx_bits, r), hb = ldp(indptr, idx_bits, r + 1);
  if (hb - lb <= DGNN_SEG) return;
  if (slot == 0 ? (lb >= cs) : (lb < cs)) return;
  const i64 e0 = lb > cs ? lb : cs, e1 = hb < ce ? hb : ce;
  float s = 0.f;
  for (i64 e = e0; e < e1; ++e) s += __ldg(grad_edge + e * H + h);
  part[(2 * j + slot) * H + h] = s;
}

__global__ void k_rowred_merge(i64 n_rows, i64 nnz, int H, const void* indptr, int idx_bits,
                               const float* part, float* grad_attn_row) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  const i64 j = t / H;
  const int h = (int)(t % H);
  const i64 cs = j * DGNN_SEG;
  if (cs >= nnz) return;
  const i64 ce = (cs + DGNN_SEG < nnz) ? cs + DGNN_SEG : nnz;
  const i64 r = find_row(indptr, idx_bits, n_rows, ce - 1);
  const i64 lb = ldp(indptr, idx_bits, r), hb = ldp(indptr, idx_bits, r + 1);
  if (hb - lb <= DGNN_SEG || lb < cs) return;
  float s = part[(2 * j + 1) * H + h];
  for (i64 jj = j + 1; jj * DGNN_SEG < hb; ++jj) s += part[(2 * jj) * H + h];
  grad_attn_row[r * H + h] = s;
}

// ---------------------------------------------------------------- host side
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline size_t up256(size_t x) { return (x + 255) & ~size_t(255); }
inline i64 up4(i64 x) { return (x + 3) & ~i64(3); }

struct FastShape {
  bool ok;
  int hf4, f4_shift, vpl, lpr;
  bool wide_ok = true;   // the row tensors of this call are 32-byte aligned (the same-head layout uses 256-bit accesses)
};
inline FastShape fast_shape(int h, int f) {
  FastShape s{false, 0, 0, 0, 32, true};
  if (f % 4) return s;
  const int sh = ilog2_exact(f / 4);
  if (sh < 0) return s;
  const i64 hf4 = (i64)h * (f / 4);
  if (hf4 > 256) return s;
  s.ok = true;
  s.hf4 = (int)hf4;
  s.f4_shift = sh;
  s.vpl = hf4 <= 32 ? 1 : hf4 <= 64 ? 2 : hf4 <= 128 ? 4 : 8;
  s.lpr = hf4 <= 8 ? 8 : hf4 <= 16 ? 16 : 32;
  return s;
}

// floats per forward partial / carried-state slot; `neg` adds the negative-side accumulators
inline i64 fwd_slot_stride(int h, int f, bool neg) {
  return neg ? 2 * (i64)h * f + up4(3 * (i64)h) : (i64)h * f + up4(2 * (i64)h);
}
inline i64 bwd_slot_stride(int h, int f) { return (i64)h * f + up4((i64)h); }

template <class Op>
int launch_fwd_op(const FastShape& fs, i64 n_rows, i64 nnz, int h, int f, const void* row_ptr, int idx_bits,
                  const int* col_ind, const float* attn_row, const float* attn_col, const float* in_feat,
                  float slope, float drop, const float* mask, float* out, float* edge_max, float* edge_sum,
                  void* ws, float* state, int first, int last, const float* bias, float* out_neg, float* a_neg,
                  const unsigned char* stage_mask, int stage, const unsigned* hot, cudaStream_t s) {
  Op op;
  op.n_rows = n_rows; op.nnz = nnz; op.indptr = row_ptr; op.idx_bits = idx_bits;
  op.H = h; op.hf4 = fs.hf4; op.f4_shift = fs.f4_shift;
  op.col_ind = col_ind; op.attn_row = attn_row; op.attn_col = attn_col;
  op.in_feat = reinterpret_cast<const float4*>(in_feat); op.mask = mask;
  op.slope = slope; op.drop_p = drop; op.inv_keep = (float)(1.0 / (1.0 - (double)drop));
  op.out = reinterpret_cast<float4*>(out); op.edge_max = edge_max; op.edge_sum = edge_sum;
  op.ws = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + DGNN_WS_HEADER);
  op.slot_stride = fwd_slot_stride(h, f, out_neg != nullptr);
  op.state = state; op.first = first; op.last = last; op.skip_empty = (!first && !last && !stage_mask) ? 1 : 0;
  op.stage_mask = stage_mask; op.stage = stage;
  op.bias = reinterpret_cast<const float4*>(bias);
  op.out_neg = reinterpret_cast<float4*>(out_neg); op.a_neg = a_neg;
  op.hot = hot;
  return dgnn_launch_trio(op, reinterpret_cast<unsigned long long*>(ws), s);
}

// Rows of more than 32 vectors whose heads hold at least VPL vectors use the same-head lane
// layout (gat_sh.cuh); everything else the plain one.
inline bool same_head_layout(const FastShape& fs) { return fs.wide_ok && fs.vpl > 1 && (1 << fs.f4_shift) >= fs.vpl; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }

// use_hot selects the kernel variant with the second (evict_last) load path; it exists without a dropout mask only
template <int VPL, bool MASK, bool FULL, int LPR, bool NEG, class... A>
int launch_fwd(bool use_hot, const FastShape& fs, A... a) {
  if constexpr (VPL > 1) {
    if (same_head_layout(fs)) {
      if constexpr (!MASK && NEG) {
        if (use_hot) return launch_fwd_op<GatFwdOpSH<VPL, MASK, FULL, NEG, true>>(fs, a...);
      }
      return launch_fwd_op<GatFwdOpSH<VPL, MASK, FULL, NEG>>(fs, a...);
    }
  }
  return launch_fwd_op<GatFwdOp<VPL, MASK, FULL, LPR, NEG>>(fs, a...);
}

template <class Op>
int launch_bwd_op(const FastShape& fs, i64 n_cols, i64 nnz, int h, int f, const void* col_ptr, int idx_bits,
                  const int* row_ind, const int* permute, const float* pack, const float* mask,
                  const float* in_feat, const float* attn_col, const float* grad_out, float slope, float drop,
                  float* grad_feat, float* grad_attn_col, float* grad_edge, float* ws, unsigned long long* counter,
                  float* state, int first, int last, const unsigned char* stage_mask, int stage, const unsigned* hot,
                  cudaStream_t s) {
  Op op;
  op.n_rows = n_cols; op.nnz = nnz; op.indptr = col_ptr; op.idx_bits = idx_bits;
  op.H = h; op.hf4 = fs.hf4; op.f4_shift = fs.f4_shift;
  op.row_ind = row_ind; op.permute = permute; op.pack = reinterpret_cast<const float4*>(pack);
  op.mask = mask; op.in_feat = reinterpret_cast<const float4*>(in_feat); op.attn_col = attn_col;
  op.grad_out = reinterpret_cast<const float4*>(grad_out);
  op.slope = slope; op.drop_p = drop; op.inv_keep = (float)(1.0 / (1.0 - (double)drop));
  op.grad_feat = reinterpret_cast<float4*>(grad_feat); op.grad_attn_col = grad_attn_col;
  op.grad_edge = grad_edge; op.ws = ws; op.slot_stride = bwd_slot_stride(h, f);
  op.state = state; op.first = first; op.last = last; op.skip_empty = (!first && !last && !stage_mask) ? 1 : 0;
  op.stage_mask = stage_mask; op.stage = stage;
  op.hot = hot;
  return dgnn_launch_trio(op, counter, s);
}

template <int VPL, bool MASK, bool FULL, int LPR, bool EDGE, class... A>
int launch_bwd(bool use_hot, const FastShape& fs, A... a) {
  if constexpr (VPL > 1) {
    if (same_head_layout(fs)) {
      if constexpr (!MASK && !EDGE) {
        if (use_hot) return launch_bwd_op<GatBwdOpSH<VPL, MASK, FULL, EDGE, true>>(fs, a...);
      }
      return launch_bwd_op<GatBwdOpSH<VPL, MASK, FULL, EDGE>>(fs, a...);
    }
  }
  return launch_bwd_op<GatBwdOp<VPL, MASK, FULL, LPR>>(fs, a...);
}

// FULL = the row is exactly LPR*VPL float4 vectors wide: no lane is ever idle.
// LPR (lanes per row) is 32 except for rows of at most 16 / 8 vectors.
#define DGNN_DISPATCH_VM(V, L, MASKED, FULLW, CALL)                                          \
  return MASKED ? (FULLW ? CALL(V, true, true, L) : CALL(V, true, false, L))                 \
                : (FULLW ? CALL(V, false, true, L) : CALL(V, false, false, L));
#define DGNN_DISPATCH_VPL(vpl, lpr, MASKED, FULLW, CALL)             \
  switch (vpl) {                                                     \
    case 1:                                                          \
      if (lpr == 8) { DGNN_DISPATCH_VM(1, 8, MASKED, FULLW, CALL) }  \
      if (lpr == 16) { DGNN_DISPATCH_VM(1, 16, MASKED, FULLW, CALL) }\
      DGNN_DISPATCH_VM(1, 32, MASKED, FULLW, CALL)                   \
    case 2: DGNN_DISPATCH_VM(2, 32, MASKED, FULLW, CALL)             \
    case 4: DGNN_DISPATCH_VM(4, 32, MASKED, FULLW, CALL)             \
    default: DGNN_DISPATCH_VM(8, 32, MASKED, FULLW, CALL)            \
  }

struct BwdLayout {
  size_t counter, grad_edge, col_part, row_part, pack, total;
};
// `edge`: room for the per-edge term d_e and the long-row partials of its row reduction (only the entry
// points that return grad_attn_row from the column pass need them)
inline BwdLayout bwd_layout(i64 n_rows, i64 nnz, int h, int f, bool edge) {
  BwdLayout L;
  const i64 nc = dgnn_num_chunks(nnz);
  size_t off = 0;
  L.counter = off;   off += DGNN_WS_HEADER;
  L.grad_edge = off; off += edge ? up256((size_t)nnz * h * sizeof(float)) : 0;
  L.col_part = off;  off += up256((size_t)(2 * nc) * bwd_slot_stride(h, f) * sizeof(float));
  L.row_part = off;  off += edge ? up256((size_t)(2 * nc) * h * sizeof(float)) : 0;
  L.pack = off;      off += edge ? up256((size_t)n_rows * h * 4 * sizeof(float)) : 0;
  L.total = off + 256;
  return L;
}

int check_common(i64 n, i64 nnz, int h, int f, int idx_bits) {
  if (n < 0 || nnz < 0 || h <= 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (idx_bits != 32 && idx_bits != 64) return DGNN_ERR_IDX_BITS;
  if (idx_bits == 32 && nnz > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (n > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;  // node ids are int32
  return DGNN_OK;
}

}  // namespace

extern "C" {

int dgnn_gat_fast_shape(int h, int f) { return (h > 0 && f > 0 && fast_shape(h, f).ok) ? 1 : 0; }

size_t dgnn_gat_forward_workspace_bytes(int64_t n_rows, int64_t nnz, int h, int f) {
  (void)n_rows;
  if (nnz <= DGNN_SEG || h <= 0 || f <= 0) return DGNN_WS_HEADER;
  return DGNN_WS_HEADER + up256((size_t)(2 * dgnn_num_chunks(nnz)) * fwd_slot_stride(h, f, true) * sizeof(float));
}

size_t dgnn_gat_forward_state_bytes(int64_t n_rows, int h, int f) {
  if (n_rows < 0 || h <= 0 || f <= 0) return 0;
  return (size_t)n_rows * fwd_slot_stride(h, f, true) * sizeof(float);
}
size_t dgnn_gat_backward_state_bytes(int64_t n_cols, int h, int f) {
  if (n_cols < 0 || h <= 0 || f <= 0) return 0;
  return (size_t)n_cols * bwd_slot_stride(h, f) * sizeof(float);
}

int dgnn_gat_forward(int64_t n_rows, int64_t nnz, int h, int f, const void* row_ptr, int idx_bits,
                     const int32_t* col_ind, const float* attn_row, const float* attn_col,
                     const float* in_feat, float negative_slope, float attn_drop, const float* edge_mask,
                     float* out, float* edge_max, float* edge_sum, void* workspace,
                     size_t workspace_bytes, void* stream) {
  return dgnn_gat_forward_staged(n_rows, nnz, h, f, row_ptr, idx_bits, col_ind, attn_row, attn_col, in_feat,
                                 negative_slope, attn_drop, edge_mask, nullptr, out, edge_max, edge_sum, nullptr,
                                 nullptr, nullptr, 1, 1, nullptr, 0, nullptr, workspace, workspace_bytes, stream);
}

int dgnn_gat_forward_staged(int64_t n_rows, int64_t nnz, int h, int f, const void* row_ptr, int idx_bits,
                            const int32_t* col_ind, const float* attn_row, const float* attn_col,
                            const float* in_feat, float negative_slope, float attn_drop,
                            const float* edge_mask, const float* bias, float* out, float* edge_max,
                            float* edge_sum, float* out_neg, float* a_neg, float* state, int first, int last,
                            const uint8_t* stage_mask, int stage, const uint32_t* hot_cols,
                            void* workspace, size_t workspace_bytes, void* stream) {
  int st = check_common(n_rows, nnz, h, f, idx_bits);
  if (st) return st;
  const bool staged = !(first && last);
  if (stage_mask && (stage < 0 || stage > 7)) return DGNN_ERR_VALUE;
  // with a stage mask rows are written out in whatever stage is their last: the outputs are needed in every stage
  const bool need_out = last || stage_mask != nullptr;
  if (staged && (!state || !aligned16(state))) return state ? DGNN_ERR_ALIGN : DGNN_ERR_NULL;
  if (!(attn_drop >= 0.f && attn_drop < 1.f)) return DGNN_ERR_VALUE;
  if ((out_neg == nullptr) != (a_neg == nullptr)) return DGNN_ERR_NULL;
  if (n_rows == 0) return DGNN_OK;
  if (!row_ptr || !attn_row || (need_out && !out) || (nnz > 0 && (!col_ind || !attn_col || !in_feat))) return DGNN_ERR_NULL;
  if ((edge_max == nullptr) != (edge_sum == nullptr)) return DGNN_ERR_NULL;
  if (attn_drop > 0.f && !edge_mask) return DGNN_ERR_NULL;
  const float* mask = attn_drop > 0.f ? edge_mask : nullptr;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FastShape fs = fast_shape(h, f);
  fs.wide_ok = aligned32(in_feat);   // the gathered tensor; results check their own alignment when they are stored
  if (fs.ok && aligned16(in_feat) && aligned16(out) && aligned16(bias) && aligned16(out_neg)) {
    if (!workspace || workspace_bytes < dgnn_gat_forward_workspace_bytes(n_rows, nnz, h, f))
      return DGNN_ERR_WORKSPACE;
    if (!aligned16(workspace)) return DGNN_ERR_ALIGN;
#define FWD_ARGS                                                                                             \
  fs, n_rows, nnz, h, f, row_ptr, idx_bits, col_ind, attn_row, attn_col, in_feat, negative_slope, attn_drop, \
      mask, out, edge_max, edge_sum, workspace, state, first, last, bias, out_neg, a_neg, stage_mask, stage, \
      hot_cols, s
#define CALL_FWD(V, M, FW, L) \
  (out_neg ? launch_fwd<V, M, FW, L, true>(hot_cols != nullptr, FWD_ARGS) : launch_fwd<V, M, FW, L, false>(false, FWD_ARGS))
    DGNN_DISPATCH_VPL(fs.vpl, fs.lpr, mask != nullptr, fs.hf4 == fs.lpr * fs.vpl, CALL_FWD)
#undef CALL_FWD
#undef FWD_ARGS
  }
  // staged sweeps, the bias epilogue and the negative-side outputs exist only for the float4 layout
  if (staged || bias || out_neg || stage_mask) return DGNN_ERR_SHAPE;
  k_gat_fwd_generic<<<dgnn_grid(n_rows * h, DGNN_WARPS), DGNN_THREADS, 0, s>>>(
      n_rows, h, f, row_ptr, idx_bits, col_ind, attn_row, attn_col, in_feat, mask, negative_slope,
      attn_drop, (float)(1.0 / (1.0 - (double)attn_drop)), out, edge_max, edge_sum);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_gat_rowstat(int64_t n_rows, int h, int f, const float* attn_row, const float* edge_max,
                     const float* edge_sum, const float* out, const float* grad_out, float* pack,
                     void* stream) {
  if (n_rows < 0 || h <= 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (n_rows == 0) return DGNN_OK;
  if (!attn_row || !edge_max || !edge_sum || !out || !grad_out || !pack) return DGNN_ERR_NULL;
  if (!aligned16(pack)) return DGNN_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const FastShape fs = fast_shape(h, f);
  float4* pk = reinterpret_cast<float4*>(pack);
  if (fs.ok && aligned16(out) && aligned16(grad_out)) {
    const float4* o4 = reinterpret_cast<const float4*>(out);
    const float4* g4 = reinterpret_cast<const float4*>(grad_out);
    const unsigned grid = dgnn_grid(n_rows, DGNN_WARPS);
    switch (fs.vpl) {
      case 1: k_gat_rowstat<1><<<grid, DGNN_THREADS, 0, s>>>(n_rows, h, fs.hf4, fs.f4_shift, attn_row, edge_max, edge_sum, o4, g4, pk); break;
      case 2: k_gat_rowstat<2><<<grid, DGNN_THREADS, 0, s>>>(n_rows, h, fs.hf4, fs.f4_shift, attn_row, edge_max, edge_sum, o4, g4, pk); break;
      case 4: k_gat_rowstat<4><<<grid, DGNN_THREADS, 0, s>>>(n_rows, h, fs.hf4, fs.f4_shift, attn_row, edge_max, edge_sum, o4, g4, pk); break;
      default: k_gat_rowstat<8><<<grid, DGNN_THREADS, 0, s>>>(n_rows, h, fs.hf4, fs.f4_shift, attn_row, edge_max, edge_sum, o4, g4, pk); break;
    }
  } else {
    k_gat_rowstat_generic<<<dgnn_grid(n_rows * h, DGNN_WARPS), DGNN_THREADS, 0, s>>>(
        n_rows, h, f, attn_row, edge_max, edge_sum, out, grad_out, pk);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

size_t dgnn_gat_rowstat_bias_workspace_bytes(int h, int f) {
  if (h <= 0 || f <= 0) return 256;
  return up256((size_t)148 * 8 * h * f * sizeof(float)) + 256;    // room for up to 1184 CTAs
}

int dgnn_gat_rowstat_full(int64_t n_rows, int h, int f, const float* attn_row, const float* edge_max,
                          const float* edge_sum, const float* out, const float* grad_out, const float* bias,
                          const float* out_neg, const float* a_neg, float negative_slope, float* pack,
                          float* grad_attn_row, float* grad_bias, float* grad_copy, const int32_t* send_ptr,
                          const int32_t* send_pos, float* send_grad, float* send_pack, void* workspace,
                          size_t workspace_bytes, void* stream) {
  if (n_rows < 0 || h <= 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (send_ptr && (!send_pos || !send_grad || !send_pack)) return DGNN_ERR_NULL;
  if (send_ptr && (!aligned16(send_grad) || !aligned16(send_pack))) return DGNN_ERR_ALIGN;
  const RowFan fan{send_ptr, send_pos, reinterpret_cast<float4*>(send_grad), reinterpret_cast<float4*>(send_pack)};
  if ((bias == nullptr) != (grad_bias == nullptr)) return DGNN_ERR_NULL;
  if ((out_neg == nullptr) != (a_neg == nullptr) || (out_neg == nullptr) != (grad_attn_row == nullptr)) return DGNN_ERR_NULL;
  if (n_rows > 0 && (!attn_row || !edge_max || !edge_sum || !out || !grad_out || !pack)) return DGNN_ERR_NULL;
  const FastShape fs = fast_shape(h, f);
  if (!fs.ok) return DGNN_ERR_SHAPE;
  if (!aligned16(pack) || !aligned16(out) || !aligned16(grad_out) || !aligned16(bias) || !aligned16(grad_bias) ||
      !aligned16(out_neg) || !aligned16(grad_copy))
    return DGNN_ERR_ALIGN;
  if (bias && (!workspace || workspace_bytes < dgnn_gat_rowstat_bias_workspace_bytes(h, f))) return DGNN_ERR_WORKSPACE;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float4* part = bias ? reinterpret_cast<float4*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255)) : nullptr;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  i64 ctas = (i64)sms * 8;
  if (ctas > 148 * 8) ctas = 148 * 8;
  const i64 need = (n_rows + DGNN_WARPS - 1) / DGNN_WARPS;
  if (need < ctas) ctas = need < 1 ? 1 : need;
  const size_t smem = (size_t)DGNN_WARPS * fs.hf4 * sizeof(float4);   // <= 32 KB
  const float4* o4 = reinterpret_cast<const float4*>(out);
  const float4* g4 = reinterpret_cast<const float4*>(grad_out);
  const float4* b4 = reinterpret_cast<const float4*>(bias);
  const float4* n4 = reinterpret_cast<const float4*>(out_neg);
  float4* pk = reinterpret_cast<float4*>(pack);
  float4* gc4 = reinterpret_cast<float4*>(grad_copy);
  const float oms = 1.f - negative_slope;
#define ROWSTAT(V)                                                                                              \
  k_gat_rowstat_full<V><<<(unsigned)ctas, DGNN_THREADS, smem, s>>>(n_rows, h, fs.hf4, fs.f4_shift, attn_row,     \
      edge_max, edge_sum, o4, g4, b4, n4, a_neg, oms, pk, grad_attn_row, gc4, part, fan)
  switch (fs.vpl) {
    case 1: ROWSTAT(1); break;
    case 2: ROWSTAT(2); break;
    case 4: ROWSTAT(4); break;
    default: ROWSTAT(8); break;
  }
#undef ROWSTAT
  if (bias) k_bias_grad_final<<<dgnn_grid(fs.hf4, 128), 128, 0, s>>>((int)ctas, fs.hf4, part, reinterpret_cast<float4*>(grad_bias));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_gat_rowstat_bias(int64_t n_rows, int h, int f, const float* attn_row, const float* edge_max,
                          const float* edge_sum, const float* out, const float* grad_out, const float* bias,
                          float* pack, float* grad_bias, void* workspace, size_t workspace_bytes, void* stream) {
  if (!bias || !grad_bias) return DGNN_ERR_NULL;
  return dgnn_gat_rowstat_full(n_rows, h, f, attn_row, edge_max, edge_sum, out, grad_out, bias, nullptr, nullptr, 0.f,
                               pack, nullptr, grad_bias, nullptr, nullptr, nullptr, nullptr, nullptr, workspace,
                               workspace_bytes, stream);
}

size_t dgnn_gat_backward_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz, int h, int f) {
  (void)n_cols;
  if (n_rows < 0 || nnz < 0 || h <= 0 || f <= 0) return 256;
  return bwd_layout(n_rows, nnz, h, f, true).total;
}

size_t dgnn_gat_backward_cols_workspace_bytes(int64_t nnz, int h, int f, int with_grad_attn_row) {
  if (nnz < 0 || h <= 0 || f <= 0) return 256;
  return bwd_layout(0, nnz, h, f, with_grad_attn_row != 0).total;
}

int dgnn_gat_backward_cols(int64_t n_rows, int64_t n_cols, int64_t nnz, int h, int f, const void* row_ptr,
                           const void* col_ptr, int idx_bits, const int32_t* row_ind,
                           const int32_t* permute, const float* pack, const float* edge_mask,
                           const float* in_feat, const float* attn_col, const float* grad_out,
                           float negative_slope, float attn_drop, float* grad_feat, float* grad_attn_row,
                           float* grad_attn_col, void* workspace, size_t workspace_bytes, void* stream) {
  return dgnn_gat_backward_cols_staged(n_rows, n_cols, nnz, h, f, row_ptr, col_ptr, idx_bits, row_ind, permute, pack,
                                       edge_mask, in_feat, attn_col, grad_out, negative_slope, attn_drop, grad_feat,
                                       grad_attn_row, grad_attn_col, nullptr, 1, 1, nullptr, 0, nullptr, workspace, workspace_bytes,
                                       stream);
}

int dgnn_gat_backward_cols_staged(int64_t n_rows, int64_t n_cols, int64_t nnz, int h, int f, const void* row_ptr,
                                  const void* col_ptr, int idx_bits, const int32_t* row_ind,
                                  const int32_t* permute, const float* pack, const float* edge_mask,
                                  const float* in_feat, const float* attn_col, const float* grad_out,
                                  float negative_slope, float attn_drop, float* grad_feat, float* grad_attn_row,
                                  float* grad_attn_col, float* state, int first, int last, const uint8_t* stage_mask,
                                  int stage, const uint32_t* hot_rows, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  int st = check_common(n_rows, nnz, h, f, idx_bits);
  if (st) return st;
  const bool staged = !(first && last);
  if (stage_mask && (stage < 0 || stage > 7)) return DGNN_ERR_VALUE;
  const bool need_out = last || stage_mask != nullptr;   // with a stage mask columns are written out in their own last stage
  if (staged && (!state || !aligned16(state))) return state ? DGNN_ERR_ALIGN : DGNN_ERR_NULL;
  st = check_common(n_cols, nnz, h, f, idx_bits);
  if (st) return st;
  if (nnz > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;  // CSR / CSC positions are int32
  if (!(attn_drop >= 0.f && attn_drop < 1.f)) return DGNN_ERR_VALUE;
  const bool edge = grad_attn_row != nullptr;   // the per-edge term and its row reduction are wanted
  if (!col_ptr || (edge && !row_ptr)) return DGNN_ERR_NULL;
  if (n_cols > 0 && (!in_feat || !attn_col || (need_out && (!grad_feat || !grad_attn_col)))) return DGNN_ERR_NULL;
  if (n_rows > 0 && (!pack || !grad_out)) return DGNN_ERR_NULL;
  if (nnz > 0 && (!row_ind || (edge && !permute))) return DGNN_ERR_NULL;
  if (attn_drop > 0.f && !edge_mask) return DGNN_ERR_NULL;
  const BwdLayout L = bwd_layout(n_rows, nnz, h, f, edge);
  if (!workspace || workspace_bytes < bwd_layout(0, nnz, h, f, edge).total) return DGNN_ERR_WORKSPACE;
  if (!aligned16(pack)) return DGNN_ERR_ALIGN;
  char* wsb = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  float* grad_edge = edge ? reinterpret_cast<float*>(wsb + L.grad_edge) : nullptr;
  float* col_part = reinterpret_cast<float*>(wsb + L.col_part);
  float* row_part = reinterpret_cast<float*>(wsb + L.row_part);
  unsigned long long* counter = reinterpret_cast<unsigned long long*>(wsb + L.counter);
  const float* mask = attn_drop > 0.f ? edge_mask : nullptr;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FastShape fs = fast_shape(h, f);
  fs.wide_ok = aligned32(in_feat) && aligned32(grad_out);
  if (n_cols > 0) {
    if (fs.ok && aligned16(in_feat) && aligned16(grad_out) && aligned16(grad_feat)) {
      int rc;
#define BWD_ARGS                                                                                          \
  fs, n_cols, nnz, h, f, col_ptr, idx_bits, row_ind, permute, pack, mask, in_feat, attn_col, grad_out,   \
      negative_slope, attn_drop, grad_feat, grad_attn_col, grad_edge, col_part, counter, state, first, last, stage_mask, \
      stage, hot_rows, s
#define CALL_BWD(V, M, FW, L) \
  (edge ? launch_bwd<V, M, FW, L, true>(false, BWD_ARGS) : launch_bwd<V, M, FW, L, false>(hot_rows != nullptr, BWD_ARGS))
      auto run = [&]() -> int { DGNN_DISPATCH_VPL(fs.vpl, fs.lpr, mask != nullptr, fs.hf4 == fs.lpr * fs.vpl, CALL_BWD) };
#undef CALL_BWD
#undef BWD_ARGS
      rc = run();
      if (rc) return rc;
    } else {
      if (staged || stage_mask) return DGNN_ERR_SHAPE;
      k_gat_bwd_cols_generic<<<dgnn_grid(n_cols * h, DGNN_WARPS), DGNN_THREADS, 0, s>>>(
          n_cols, h, f, col_ptr, idx_bits, row_ind, permute, reinterpret_cast<const float4*>(pack), mask,
          in_feat, attn_col, grad_out, negative_slope, attn_drop,
          (float)(1.0 / (1.0 - (double)attn_drop)), grad_feat, grad_attn_col, grad_edge);
    }
  }
  if (edge && n_rows > 0) {
    const int tb = 256;
    const int small = nnz <= DGNN_SMALL_NNZ ? 1 : 0;   // same rule as the feature kernels: one launch for small graphs
    k_rowred_rows<<<dgnn_grid(n_rows * h, tb), tb, 0, s>>>(n_rows, h, row_ptr, idx_bits, grad_edge, grad_attn_row, small);
    if (nnz > DGNN_SEG && !small) {
      const i64 nc = dgnn_num_chunks(nnz);
      k_rowred_chunks<<<dgnn_grid(2 * nc * h, tb), tb, 0, s>>>(n_rows, nnz, h, row_ptr, idx_bits, grad_edge, row_part);
      k_rowred_merge<<<dgnn_grid(nc * h, tb), tb, 0, s>>>(n_rows, nnz, h, row_ptr, idx_bits, row_part, grad_attn_row);
    }
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_gat_backward(int64_t n, int64_t nnz, int h, int f, const void* row_ptr, const void* col_ptr,
                      int idx_bits, const int32_t* row_ind, const int32_t* permute, const float* edge_max,
                      const float* edge_sum, const float* edge_mask, const float* in_feat, const float* out,
                      const float* attn_row, const float* attn_col, const float* grad_out,
                      float negative_slope, float attn_drop, float* grad_feat, float* grad_attn_row,
                      float* grad_attn_col, void* workspace, size_t workspace_bytes, void* stream) {
  int st = check_common(n, nnz, h, f, idx_bits);
  if (st) return st;
  if (n == 0) return DGNN_OK;
  if (!grad_attn_row) return DGNN_ERR_NULL;
  const BwdLayout L = bwd_layout(n, nnz, h, f, true);
  if (!workspace || workspace_bytes < L.total) return DGNN_ERR_WORKSPACE;
  char* wsb = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  float* pack = reinterpret_cast<float*>(wsb + L.pack);
  st = dgnn_gat_rowstat(n, h, f, attn_row, edge_max, edge_sum, out, grad_out, pack, stream);
  if (st) return st;
  return dgnn_gat_backward_cols(n, n, nnz, h, f, row_ptr, col_ptr, idx_bits, row_ind, permute, pack, edge_mask,
                                in_feat, attn_col, grad_out, negative_slope, attn_drop, grad_feat,
                                grad_attn_row, grad_attn_col, workspace, workspace_bytes, stream);
}

}  // extern "C"

// "Same-head" lane layout for the fused GAT forward / backward operators.
//
// A row of H*F floats is HF4 float4 vectors, VPL per lane.  In the plain layout lane l
// owns vectors l, l+32, ... which usually belong to VPL different heads, so every
// per-head scalar (score, exp, softmax weight, SDDMM reduction) is computed VPL times
// per lane.  When a head holds at least VPL vectors (VPL divides F/4) the vectors can be
// dealt out so that all VPL vectors of a lane lie in ONE head: the head's F/4 vectors go
// to LPH = F/(4*VPL) neighbouring lanes, lane j of the head taking vectors j, j+LPH, ...
// Every load instruction then still reads LPH*16 contiguous bytes per head, while the
// per-head work drops to one score / exp / weight per lane and edge and the SDDMM
// reduction to log2(LPH) shuffles (2 instead of 6 per edge at 8 heads x 32).
#pragma once
#include "common.cuh"

// resident CTAs per SM asked of the compiler for the 2-vectors-per-lane kernels (it caps the registers per thread)
#ifndef DGNN_SH_FWD_BLOCKS
#define DGNN_SH_FWD_BLOCKS 6
#endif
// 1: a lane's vectors come in neighbouring pairs (32 contiguous bytes) that are loaded and stored by one 256-bit
// instruction each; the tensors the same-head operators touch that way must then be 32-byte aligned (the launcher
// falls back to the plain layout otherwise).  0: vectors j, j + LPH, ... and 128-bit accesses.
#ifndef DGNN_LD256
#define DGNN_LD256 1
#endif
#ifndef DGNN_SH_BWD_BLOCKS
#define DGNN_SH_BWD_BLOCKS 6
#endif

template <int VPL> struct Log2;
template <> struct Log2<2> { static constexpr int v = 1; };
template <> struct Log2<4> { static constexpr int v = 2; };
template <> struct Log2<8> { static constexpr int v = 3; };

template <int VPL>
struct HeadLanes {
  int hd;         // head of this lane
  bool act;       // lane holds part of a head
  bool lead;      // first lane of its head: writes the per-head scalars
  int q[VPL];     // vectors of this lane
  int lph_shift;  // log2(lanes per head)
  __device__ __forceinline__ void init(int lane, int H, int f4_shift) {
    lph_shift = f4_shift - Log2<VPL>::v;
    const int hl = lane >> lph_shift, j = lane & ((1 << lph_shift) - 1);
    act = hl < H;
    hd = act ? hl : 0;
    lead = act && j == 0;
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      q[v] = DGNN_LD256 ? (hd << f4_shift) + ((v >> 1) << (lph_shift + 1)) + 2 * j + (v & 1)   // pairs (2j, 2j+1), then + 2*LPH
                        : (hd << f4_shift) + (v << lph_shift) + j;
  }
};

// sum d[u] over the lanes of the head (uniform, all lanes take part)
template <int U>
__device__ __forceinline__ void lanes_reduce(float (&d)[U], int lph_shift) {
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    if (s < lph_shift) {
#pragma unroll
      for (int u = 0; u < U; ++u) d[u] += __shfl_xor_sync(DGNN_FULL, d[u], 1 << s);
    }
  }
}

// the lane's VPL vectors of one gathered row (zero when !ok); KEEP: with the L2 evict_last policy `pol`
template <bool KEEP, int VPL>
__device__ __forceinline__ void load_row(float4 (&x)[VPL], const float4* row, const HeadLanes<VPL>& lm, bool ok,
                                         unsigned long long pol) {
#if DGNN_LD256
#pragma unroll
  for (int v = 0; v < VPL; v += 2) {
    if (!ok) { x[v] = zero4(); x[v + 1] = zero4(); }
    else if (KEEP) ld8_keep(row + lm.q[v], x[v], x[v + 1], pol);
    else ld8_gather(row + lm.q[v], x[v], x[v + 1]);
  }
#else
#pragma unroll
  for (int v = 0; v < VPL; ++v) x[v] = !ok ? zero4() : (KEEP ? ld4_keep(row + lm.q[v], pol) : ld4_gather(row + lm.q[v]));
#endif
}
// the lane's vectors of one result row
template <int VPL>
__device__ __forceinline__ void store_row(float4* row, const HeadLanes<VPL>& lm, const float4 (&a)[VPL]) {
#if DGNN_LD256
  if ((reinterpret_cast<uintptr_t>(row) & 31) == 0) {      // once per row; the same answer for every row of a tensor
#pragma unroll
    for (int v = 0; v < VPL; v += 2) st8(row + lm.q[v], a[v], a[v + 1]);
  } else {
#pragma unroll
    for (int v = 0; v < VPL; ++v) row[lm.q[v]] = a[v];
  }
#else
#pragma unroll
  for (int v = 0; v < VPL; ++v) st4_stream(row + lm.q[v], a[v]);
#endif
}

// ------------------------------------------------------------------ forward
// NEG: also accumulate the part of the row's result that comes from edges on the negative side of
// the LeakyReLU (out_neg, a_neg); the backward derives grad_attn_row from it without a per-edge array.
// HOT: the kernel variant that honours the hot-column set (two load paths per edge); without it the set is ignored
template <int VPL, bool MASK, bool FULL, bool NEG, bool HOT = false>
struct GatFwdOpSH {
  static constexpr int MIN_BLOCKS = VPL <= 2 ? DGNN_SH_FWD_BLOCKS : (VPL == 4 ? 4 : 2);
  static constexpr bool HAS_PARTIALS = true;
  static constexpr int U = VPL <= 2 ? 4 : 2;
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
  i64 slot_stride;
  float* state;
  int first, last, skip_empty;
  static constexpr bool STAGED = true;
  const unsigned char* stage_mask;   // per row: bit p set = the row has entries in stage p (NULL: every row in every stage)
  int stage;
  const float4* bias;
  float4* out_neg;
  float* a_neg;
  const unsigned* hot;   // NULL, or one bit per column: its in_feat / attn_col rows stay in the L2 (ld4_keep)

  struct State {
    HeadLanes<VPL> lm;
    float ar, m, z, zn;
    float4 acc[VPL];
    float4 accn[NEG ? VPL : 1];
  };

  __device__ __forceinline__ void init(State& st, i64 r, int lane) const {
    st.lm.init(lane, H, f4_shift);
    st.ar = st.lm.act ? __ldg(attn_row + r * H + st.lm.hd) : 0.f;
    st.m = DGNN_NEG_INIT;
    st.z = 0.f;
    st.zn = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) st.acc[v] = zero4();
    if (NEG) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) st.accn[v] = zero4();
    }
  }
  __device__ __forceinline__ void resume(State& st, i64 r, int lane, bool first_) const {
    if (!first_) merge_partial(st, state + r * slot_stride, lane);
  }
  __device__ __forceinline__ void combine(State&, int) const {}

  template <bool ALL>
  __device__ __forceinline__ void batch(State& st, int my_c, i64 ebase, int k, int cnt) const {
    int c[U];
#pragma unroll
    for (int u = 0; u < U; ++u) c[u] = __shfl_sync(DGNN_FULL, my_c, (k + u) & 31);
    float s[U];
    float4 x[U][VPL];
    bool keep[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = (ALL || k + u < cnt) && (FULL || st.lm.act);
      const bool hot_u = HOT && c[u] < 0;                       // the same for every lane: a uniform branch
      const i64 cc = c[u] & 0x7fffffff;
      keep[u] = ok;
      if (MASK) keep[u] = ok ? (__ldg(mask + (ebase + k + u) * H + st.lm.hd) > drop_p) : false;
      if (hot_u) {
        const unsigned long long pol = l2_keep_policy();   // made where it is used: no register held across the loop
        s[u] = ok ? ld1_keep(attn_col + cc * H + st.lm.hd, pol) : 0.f;
        load_row<true>(x[u], in_feat + cc * hf4, st.lm, ok, pol);
      } else {
        s[u] = ok ? __ldg(attn_col + cc * H + st.lm.hd) : 0.f;
        load_row<false>(x[u], in_feat + cc * hf4, st.lm, ok, 0ull);
      }
    }
    float l[U];
    float bm = st.m;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      l[u] = (ALL || k + u < cnt) ? leaky(st.ar + s[u], slope) : DGNN_NEG_INIT;
      bm = fmaxf(bm, l[u]);
    }
    // after the first few edges of a row the running maximum rarely moves: rescale only when it did
    // for some head of the warp (a lane whose maximum stayed multiplies by exp(0) = 1, as before)
    const bool moved = __any_sync(DGNN_FULL, bm > st.m);
    if (!FULL && !st.lm.act) { st.m = bm; return; }
    if (moved) {
      const float sc = fast_exp(st.m - bm);
      st.z *= sc;
#pragma unroll
      for (int v = 0; v < VPL; ++v) scale4(st.acc[v], sc);
      if (NEG) {
        st.zn *= sc;
#pragma unroll
        for (int v = 0; v < VPL; ++v) scale4(st.accn[v], sc);
      }
      st.m = bm;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ALL || k + u < cnt) {
        const float p = fast_exp(l[u] - bm);
        st.z += p;
        const float pn = l[u] < 0.f ? p : 0.f;
        if (NEG) st.zn += pn;
        if (!MASK || keep[u]) {
#pragma unroll
          for (int v = 0; v < VPL; ++v) fma4(st.acc[v], p, x[u][v]);
          if (NEG) {
#pragma unroll
            for (int v = 0; v < VPL; ++v) fma4(st.accn[v], pn, x[u][v]);
          }
        }
      }
    }
  }

  __host__ __device__ __forceinline__ int ring_bytes() const { return 0; }   // gathers go straight into registers
  __device__ __forceinline__ void range(State& st, i64, i64 e0, i64 e1, int lane, float4*) const {
    for (i64 base = e0; base < e1; base += 32) {
      const int cnt = (int)((e1 - base) < 32 ? (e1 - base) : 32);
      const int my_c = lane < cnt ? dgnn_tag_hot(HOT ? hot : nullptr, ld_index(col_ind + base + lane)) : 0;
      int k = 0;
      for (; k + U <= cnt; k += U) batch<true>(st, my_c, base, k, cnt);
      if (k < cnt) batch<false>(st, my_c, base, k, cnt);
    }
  }

  __device__ __forceinline__ void finalize(State& st, i64 r, int lane, bool last_) const {
    if (!last_) { store_partial(st, state + r * slot_stride, lane); return; }
    if (!st.lm.act) return;
    const float sc = st.z > 0.f ? inv_keep / st.z : 0.f;
    float4 res[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      res[v] = st.acc[v];
      scale4(res[v], sc);
      if (bias) add4(res[v], __ldg(bias + st.lm.q[v]));
    }
    store_row<VPL>(out + r * hf4, st.lm, res);
    if (NEG) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        res[v] = st.accn[v];
        scale4(res[v], sc);
      }
      store_row<VPL>(out_neg + r * hf4, st.lm, res);
    }
    if (st.lm.lead && edge_max) {
      edge_max[r * H + st.lm.hd] = st.m;
      edge_sum[r * H + st.lm.hd] = st.z;
    }
    if (NEG && st.lm.lead) a_neg[r * H + st.lm.hd] = st.z > 0.f ? st.zn / st.z : 0.f;
  }

  // slot layout: [acc H*F | m H | z H | (NEG: zn H) | pad to 4 | (NEG: accn H*F)]
  __device__ __forceinline__ void store_partial(State& st, float* p, int) const {
    if (!st.lm.act) return;
#pragma unroll
    for (int v = 0; v < VPL; ++v) reinterpret_cast<float4*>(p)[st.lm.q[v]] = st.acc[v];
    if (st.lm.lead) {
      p[hf4 * 4 + st.lm.hd] = st.m;
      p[hf4 * 4 + H + st.lm.hd] = st.z;
      if (NEG) p[hf4 * 4 + 2 * H + st.lm.hd] = st.zn;
    }
    if (NEG) {
      float4* pn = reinterpret_cast<float4*>(p + slot_stride - hf4 * 4);
#pragma unroll
      for (int v = 0; v < VPL; ++v) pn[st.lm.q[v]] = st.accn[v];
    }
  }

  __device__ __forceinline__ void merge_partial(State& st, const float* p, int) const {
    if (!st.lm.act) return;
    const float mi = p[hf4 * 4 + st.lm.hd];
    const float zi = p[hf4 * 4 + H + st.lm.hd];
    const float mn = fmaxf(st.m, mi);
    const float s1 = fast_exp(st.m - mn), s2 = fast_exp(mi - mn);
    st.z = st.z * s1 + zi * s2;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      scale4(st.acc[v], s1);
      fma4(st.acc[v], s2, reinterpret_cast<const float4*>(p)[st.lm.q[v]]);
    }
    if (NEG) {
      st.zn = st.zn * s1 + p[hf4 * 4 + 2 * H + st.lm.hd] * s2;
      const float4* pn = reinterpret_cast<const float4*>(p + slot_stride - hf4 * 4);
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        scale4(st.accn[v], s1);
        fma4(st.accn[v], s2, pn[st.lm.q[v]]);
      }
    }
    st.m = mn;
  }
};

// ------------------------------------------------------------ backward cols
// EDGE: the per-edge term d_e is written to grad_edge (CSR position through `permute`); without it -- the row
// gradient then comes from the row statistics -- neither array is touched unless a dropout mask needs the position
template <int VPL, bool MASK, bool FULL, bool EDGE, bool HOT = false>
struct GatBwdOpSH {
  static constexpr int MIN_BLOCKS = VPL <= 2 ? (EDGE || MASK ? 4 : DGNN_SH_BWD_BLOCKS) : (VPL == 4 ? 3 : 2);
  static constexpr bool HAS_PARTIALS = true;
  static constexpr int U = VPL <= 2 ? 4 : 2;
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
  float* state;
  int first, last, skip_empty;
  static constexpr bool STAGED = true;
  const unsigned char* stage_mask;   // per row: bit p set = the row has entries in stage p (NULL: every row in every stage)
  int stage;
  const unsigned* hot;   // NULL, or one bit per destination row: its grad_out / pack rows stay in the L2 (ld4_keep)

  struct State {
    HeadLanes<VPL> lm;
    float4 x[VPL], acc[VPL];
    float ac, gc;
  };

  __device__ __forceinline__ void init(State& st, i64 c, int lane) const {
    st.lm.init(lane, H, f4_shift);
    st.ac = st.lm.act ? __ldg(attn_col + c * H + st.lm.hd) : 0.f;
    st.gc = 0.f;
    load_row<false>(st.x, in_feat + c * hf4, st.lm, st.lm.act, 0ull);
#pragma unroll
    for (int v = 0; v < VPL; ++v) st.acc[v] = zero4();
  }
  __device__ __forceinline__ void resume(State& st, i64 c, int lane, bool first_) const {
    if (!first_) merge_partial(st, state + c * slot_stride, lane);
  }
  __device__ __forceinline__ void combine(State&, int) const {}

  template <bool ALL>
  __device__ __forceinline__ void batch(State& st, int my_r, int my_p, int k, int cnt) const {
    int r[U], pp[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      r[u] = __shfl_sync(DGNN_FULL, my_r, (k + u) & 31);
      pp[u] = (EDGE || MASK) ? __shfl_sync(DGNN_FULL, my_p, (k + u) & 31) : 0;
    }
    float4 pk[U], g4[U][VPL];
    bool keep[U];
    float d[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = (ALL || k + u < cnt) && (FULL || st.lm.act);
      const bool hot_u = HOT && r[u] < 0;                       // the same for every lane: a uniform branch
      const i64 rr = r[u] & 0x7fffffff;
      keep[u] = ok;
      if (MASK) keep[u] = ok ? (__ldg(mask + (i64)pp[u] * H + st.lm.hd) > drop_p) : false;
      if (hot_u) {
        const unsigned long long pol = l2_keep_policy();   // made where it is used: no register held across the loop
        pk[u] = ok ? ld4_keep(pack + rr * H + st.lm.hd, pol) : zero4();
        load_row<true>(g4[u], grad_out + rr * hf4, st.lm, ok, pol);
      } else {
        pk[u] = ok ? ld4(pack + rr * H + st.lm.hd) : zero4();
        load_row<false>(g4[u], grad_out + rr * hf4, st.lm, ok, 0ull);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float2 t = make_float2(0.f, 0.f);
#pragma unroll
      for (int v = 0; v < VPL; ++v) dot4_acc(t, g4[u][v], st.x[v]);
      d[u] = t.x + t.y;
    }
    lanes_reduce<U>(d, st.lm.lph_shift);  // executed by all lanes, also for slots past cnt
    if (!FULL && !st.lm.act) return;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (ALL || k + u < cnt) {
        const float l = leaky(pk[u].x + st.ac, slope);
        const float alpha = fast_exp(l - pk[u].y) * pk[u].z;   // pack.z = 1 / edge_sum
        const float kp = (!MASK || keep[u]) ? inv_keep : 0.f;
        float de = alpha * (d[u] * kp - pk[u].w);
        de = l < 0.f ? de * slope : de;
        st.gc += de;
        const float w = alpha * kp;
#pragma unroll
        for (int v = 0; v < VPL; ++v) fma4(st.acc[v], w, g4[u][v]);
        if (EDGE && st.lm.lead) grad_edge[(i64)pp[u] * H + st.lm.hd] = de;
      }
    }
  }

  __host__ __device__ __forceinline__ int ring_bytes() const { return 0; }   // gathers go straight into registers
  __device__ __forceinline__ void range(State& st, i64, i64 e0, i64 e1, int lane, float4*) const {
    for (i64 base = e0; base < e1; base += 32) {
      const int cnt = (int)((e1 - base) < 32 ? (e1 - base) : 32);
      const int my_r = lane < cnt ? dgnn_tag_hot(HOT ? hot : nullptr, ld_index(row_ind + base + lane)) : 0;
      // without a permutation the mask (if any) is laid out in CSC order: the position is the index
      int my_p = 0;
      if (EDGE || MASK) my_p = lane < cnt ? (permute ? __ldg(permute + base + lane) : (int)(base + lane)) : 0;
      int k = 0;
      for (; k + U <= cnt; k += U) batch<true>(st, my_r, my_p, k, cnt);
      if (k < cnt) batch<false>(st, my_r, my_p, k, cnt);
    }
  }

  __device__ __forceinline__ void finalize(State& st, i64 c, int lane, bool last_) const {
    if (!last_) { store_partial(st, state + c * slot_stride, lane); return; }
    if (!st.lm.act) return;
    store_row<VPL>(grad_feat + c * hf4, st.lm, st.acc);
    if (st.lm.lead) grad_attn_col[c * H + st.lm.hd] = st.gc;
  }

  __device__ __forceinline__ void store_partial(State& st, float* p, int) const {
    if (!st.lm.act) return;
#pragma unroll
    for (int v = 0; v < VPL; ++v) reinterpret_cast<float4*>(p)[st.lm.q[v]] = st.acc[v];
    if (st.lm.lead) p[hf4 * 4 + st.lm.hd] = st.gc;
  }

  __device__ __forceinline__ void merge_partial(State& st, const float* p, int) const {
    if (!st.lm.act) return;
#pragma unroll
    for (int v = 0; v < VPL; ++v) add4(st.acc[v], reinterpret_cast<const float4*>(p)[st.lm.q[v]]);
    st.gc += p[hf4 * 4 + st.lm.hd];
  }
};

// Multi-head SDDMM, multi-head transpose and the MoNet (GMM) kernels for sm_100a.
//
// SDDMM and the GMM aggregation use the same warp-per-row float4 layout and
// long-row splitting as the GAT kernels (common.cuh): the row operand stays in
// registers, each edge gathers one contiguous H*F row of the column operand.
#include "common.cuh"
#include "gat_sh.cuh"   // HeadLanes, lanes_reduce, load_row: the same-head lane layout with 256-bit gathers

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline size_t up256(size_t x) { return (x + 255) & ~size_t(255); }

struct FastShape {
  bool ok;
  int hf4, f4_shift, vpl, lpr;
  bool same_head = false;   // set per call: heads of at least vpl vectors and 32-byte aligned operands
};
inline FastShape fast_shape(int h, int f) {
  FastShape s{false, 0, 0, 0, 32, false};
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

// ------------------------------------------------------------------- SDDMM
template <int VPL, int LPR>
struct SddmmOp {
  static constexpr int EPW = 32 / LPR;
  static constexpr int MIN_BLOCKS = VPL <= 2 ? 5 : (VPL == 4 ? 4 : 2);
  static constexpr bool HAS_PARTIALS = false;   // outputs are per edge: nothing to fold
  i64 n_rows, nnz;
  const void* indptr;
  int idx_bits;
  int H, hf4, f4_shift;
  float* ws;
  i64 slot_stride;
  int skip_empty;
  const int* col_ind;
  const float4* a;
  const float4* b;
  float* out;

  struct State {
    LaneMap<VPL, LPR> lm;
    float4 a[VPL];
  };
  __device__ __forceinline__ void init(State& st, i64 r, int lane) const {
    st.lm.init(lane, hf4, f4_shift);
#pragma unroll
    for (int v = 0; v < VPL; ++v) st.a[v] = st.lm.act[v] ? ld4(a + r * hf4 + st.lm.q[v]) : zero4();
  }
  __host__ __device__ __forceinline__ int ring_bytes() const { return 0; }   // gathers go straight into registers
  __device__ __forceinline__ void range(State& st, i64, i64 e0, i64 e1, int lane, float4*) const {
    constexpr int U = VPL <= 2 ? 4 : 2;
    for (i64 base = e0; base < e1; base += 32) {
      const int cnt = (int)((e1 - base) < 32 ? (e1 - base) : 32);
      const int my_c = lane < cnt ? __ldg(col_ind + base + lane) : 0;
      for (int k = 0; k < cnt; k += U * EPW) {
        float4 x[U][VPL];
        int slot[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          slot[u] = k + u * EPW + st.lm.sg;
          const int c = __shfl_sync(DGNN_FULL, my_c, slot[u] & 31);
#pragma unroll
          for (int v = 0; v < VPL; ++v)
            x[u][v] = (slot[u] < cnt && st.lm.act[v]) ? ld4(b + (i64)c * hf4 + st.lm.q[v]) : zero4();
        }
        float d[U][VPL];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int v = 0; v < VPL; ++v) d[u][v] = dot4(st.a[v], x[u][v]);
        head_reduce<U, VPL>(d, f4_shift);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (slot[u] < cnt) {
#pragma unroll
            for (int v = 0; v < VPL; ++v)
              if (st.lm.lead[v]) out[(base + slot[u]) * H + st.lm.hd[v]] = d[u][v];
          }
        }
      }
    }
  }
  static constexpr bool STAGED = false;
  __device__ __forceinline__ void resume(State&, i64, int, bool) const {}
  __device__ __forceinline__ void combine(State&, int) const {}
  __device__ __forceinline__ void finalize(State&, i64, int, bool) const {}
  __device__ __forceinline__ void store_partial(State&, float*, int) const {}
  __device__ __forceinline__ void merge_partial(State&, const float*, int) const {}
};

// SDDMM in the same-head lane layout (gat_sh.cuh): a lane's VPL vectors lie in one head and come in neighbouring
// pairs, so the column operand is gathered with 256-bit loads, the dot product of a head needs log2(lanes per head)
// shuffles instead of log2(vectors per head) per vector, and every lane computes one head's product per edge.
// For rows of more than 32 vectors whose heads hold at least VPL vectors, 32-byte aligned operands.
template <int VPL>
struct SddmmOpSH {
  static constexpr int MIN_BLOCKS = VPL <= 2 ? 5 : (VPL == 4 ? 4 : 3);
  static constexpr bool HAS_PARTIALS = false;
  i64 n_rows, nnz;
  const void* indptr;
  int idx_bits;
  int H, hf4, f4_shift;
  float* ws;
  i64 slot_stride;
  int skip_empty;
  const int* col_ind;
  const float4* a;
  const float4* b;
  float* out;

  struct State {
    HeadLanes<VPL> lm;
    float4 a[VPL];
  };
  __device__ __forceinline__ void init(State& st, i64 r, int lane) const {
    st.lm.init(lane, H, f4_shift);
    load_row<false>(st.a, a + r * hf4, st.lm, st.lm.act, 0ull);
  }
  __host__ __device__ __forceinline__ int ring_bytes() const { return 0; }
  __device__ __forceinline__ void range(State& st, i64, i64 e0, i64 e1, int lane, float4*) const {
    constexpr int U = VPL <= 2 ? 4 : 2;
    for (i64 base = e0; base < e1; base += 32) {
      const int cnt = (int)((e1 - base) < 32 ? (e1 - base) : 32);
      const int my_c = lane < cnt ? __ldg(col_ind + base + lane) : 0;
      for (int k = 0; k < cnt; k += U) {
        float4 x[U][VPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = __shfl_sync(DGNN_FULL, my_c, (k + u) & 31);
          load_row<false>(x[u], b + (i64)c * hf4, st.lm, k + u < cnt && st.lm.act, 0ull);
        }
        float d[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float2 t = make_float2(0.f, 0.f);
#pragma unroll
          for (int v = 0; v < VPL; ++v) dot4_acc(t, st.a[v], x[u][v]);
          d[u] = t.x + t.y;
        }
        lanes_reduce<U>(d, st.lm.lph_shift);   // all lanes take part
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (k + u < cnt && st.lm.lead) out[(base + k + u) * H + st.lm.hd] = d[u];
      }
    }
  }
  static constexpr bool STAGED = false;
  __device__ __forceinline__ void resume(State&, i64, int, bool) const {}
  __device__ __forceinline__ void combine(State&, int) const {}
  __device__ __forceinline__ void finalize(State&, i64, int, bool) const {}
  __device__ __forceinline__ void store_partial(State&, float*, int) const {}
  __device__ __forceinline__ void merge_partial(State&, const float*, int) const {}
};

// any H, F: one warp per (edge-block of a row, head) -- simple and slow
__global__ void __launch_bounds__(DGNN_THREADS)
k_sddmm_generic(i64 n_rows, int H, int F, const void* indptr, int idx_bits, const int* col_ind,
                const float* a, const float* b, float* out) {
  const int lane = threadIdx.x & 31;
  const i64 w = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  if (w >= n_rows * H) return;
  const i64 r = w / H;
  const int h = (int)(w % H);
  const i64 lb = ldp(indptr, idx_bits, r), hb = ldp(indptr, idx_bits, r + 1);
  for (i64 e = lb; e < hb; ++e) {
    const i64 c = col_ind[e];
    float d = 0.f;
    for (int f = lane; f < F; f += 32) d = fmaf(__ldg(a + (r * H + h) * F + f), __ldg(b + (c * H + h) * F + f), d);
    for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(DGNN_FULL, d, o);
    if (lane == 0) out[e * H + h] = d;
  }
}

// ------------------------------------------------- single-head COO SDDMM
// out[e] = <d1[row[e], :], d2[col[e], :]> for edges in any order: one warp per edge
template <typename V>
__global__ void __launch_bounds__(DGNN_THREADS)
k_coo_sddmm(i64 nnz, int kv, const int* row, const int* col, const V* d1, const V* d2, float* out) {
  const int lane = threadIdx.x & 31;
  const i64 e = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  if (e >= nnz) return;
  const i64 r = __ldg(row + e), c = __ldg(col + e);
  float acc = 0.f;
  for (int i = lane; i < kv; i += 32) {
    if constexpr (sizeof(V) == 16) acc += dot4(__ldg(d1 + r * kv + i), __ldg(d2 + c * kv + i));
    else acc = fmaf(__ldg(d1 + r * kv + i), __ldg(d2 + c * kv + i), acc);
  }
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(DGNN_FULL, acc, o);
  if (lane == 0) out[e] = acc;
}

// --------------------------------------------------------------- transpose
__global__ void k_transpose4(i64 nnz, int h4, const int* permute, const float4* in, float4* out) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nnz * h4) return;
  const i64 i = t / h4;
  const int q = (int)(t % h4);
  out[t] = ld4(in + (i64)__ldg(permute + i) * h4 + q);
}
__global__ void k_transpose1(i64 nnz, int h, const int* permute, const float* in, float* out) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nnz * h) return;
  const i64 i = t / h;
  const int q = (int)(t % h);
  out[t] = __ldg(in + (i64)__ldg(permute + i) * h + q);
}

// --------------------------------------------------------------------- GMM
__device__ __forceinline__ float gauss_w(const float* pseudo, const float* mu, const float* sig,
                                         i64 e, int k, int dim) {
  float acc = 0.f;
  for (int d = 0; d < dim; ++d) {
    const float t = (__ldg(pseudo + e * dim + d) - __ldg(mu + k * dim + d)) * __ldg(sig + k * dim + d);
    acc = fmaf(t, t, acc);
  }
  return expf(-0.5f * acc);
}

template <int VPL, int LPR>
struct GmmOp {
  static constexpr int EPW = 32 / LPR;
  static constexpr int MIN_BLOCKS = VPL <= 2 ? 5 : (VPL == 4 ? 4 : 2);
  static constexpr bool HAS_PARTIALS = true;
  i64 n_rows, nnz;
  const void* indptr;
  int idx_bits;
  int H, hf4, f4_shift, dim;  // H = number of Gaussian kernels
  const int* col_ind;
  const float4* feat;
  const float* pseudo;
  const float* mu;
  const float* sig;
  float4* out;
  float* ws;
  i64 slot_stride;
  int skip_empty;

  struct State {
    LaneMap<VPL, LPR> lm;
    float4 acc[VPL];
  };
  __device__ __forceinline__ void init(State& st, i64, int lane) const {
    st.lm.init(lane, hf4, f4_shift);
#pragma unroll
    for (int v = 0; v < VPL; ++v) st.acc[v] = zero4();
  }
  __host__ __device__ __forceinline__ int ring_bytes() const { return 0; }   // gathers go straight into registers
  __device__ __forceinline__ void range(State& st, i64, i64 e0, i64 e1, int lane, float4*) const {
    constexpr int U = VPL <= 2 ? 4 : 2;
    for (i64 base = e0; base < e1; base += 32) {
      const int cnt = (int)((e1 - base) < 32 ? (e1 - base) : 32);
      const int my_c = lane < cnt ? __ldg(col_ind + base + lane) : 0;
      for (int k = 0; k < cnt; k += U * EPW) {
        float4 x[U][VPL];
        int slot[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          slot[u] = k + u * EPW + st.lm.sg;
          const int c = __shfl_sync(DGNN_FULL, my_c, slot[u] & 31);
#pragma unroll
          for (int v = 0; v < VPL; ++v)
            x[u][v] = (slot[u] < cnt && st.lm.act[v]) ? ld4(feat + (i64)c * hf4 + st.lm.q[v]) : zero4();
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (slot[u] < cnt) {
#pragma unroll
            for (int v = 0; v < VPL; ++v)
              if (st.lm.act[v]) fma4(st.acc[v], gauss_w(pseudo, mu, sig, base + slot[u], st.lm.hd[v], dim), x[u][v]);
          }
        }
      }
    }
  }
  static constexpr bool STAGED = false;
  __device__ __forceinline__ void resume(State&, i64, int, bool) const {}
  __device__ __forceinline__ void combine(State& st, int) const {
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) {
      float4 ao;
      ao.x = __shfl_xor_sync(DGNN_FULL, st.acc[0].x, off);
      ao.y = __shfl_xor_sync(DGNN_FULL, st.acc[0].y, off);
      ao.z = __shfl_xor_sync(DGNN_FULL, st.acc[0].z, off);
      ao.w = __shfl_xor_sync(DGNN_FULL, st.acc[0].w, off);
      const bool low = (st.lm.sg & (off / LPR)) == 0;
      float4 a = low ? st.acc[0] : ao, b = low ? ao : st.acc[0];
      add4(a, b);
      st.acc[0] = a;
    }
  }
  __device__ __forceinline__ void finalize(State& st, i64 r, int, bool) const {
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (st.lm.wr[v]) out[r * hf4 + st.lm.q[v]] = st.acc[v];
  }
  __device__ __forceinline__ void store_partial(State& st, float* pf, int) const {
    float4* p = reinterpret_cast<float4*>(pf);
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (st.lm.wr[v]) p[st.lm.q[v]] = st.acc[v];
  }
  __device__ __forceinline__ void merge_partial(State& st, const float* pf, int) const {
    const float4* p = reinterpret_cast<const float4*>(pf);
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (st.lm.act[v]) add4(st.acc[v], p[st.lm.q[v]]);
  }
};

__global__ void __launch_bounds__(DGNN_THREADS)
k_gmm_generic(i64 n_rows, int K, int dim, int F, const void* indptr, int idx_bits, const int* col_ind,
              const float* feat, const float* pseudo, const float* mu, const float* sig, float* out) {
  const int lane = threadIdx.x & 31;
  const i64 w = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  if (w >= n_rows * K) return;
  const i64 r = w / K;
  const int k = (int)(w % K);
  const i64 lb = ldp(indptr, idx_bits, r), hb = ldp(indptr, idx_bits, r + 1);
  for (int fb = lane; fb < F; fb += 32) {
    float acc = 0.f;
    for (i64 e = lb; e < hb; ++e)
      acc = fmaf(gauss_w(pseudo, mu, sig, e, k, dim), __ldg(feat + ((i64)col_ind[e] * K + k) * F + fb), acc);
    out[(r * K + k) * F + fb] = acc;
  }
}

__global__ void k_gaussian(i64 nnz, int K, int dim, const float* pseudo, const float* mu,
                           const float* sig, float* gauss) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nnz * K) return;
  gauss[t] = gauss_w(pseudo, mu, sig, t / K, (int)(t % K), dim);
}

// Gaussian backward: pseudo gradient per edge, and per-block partial sums of
// the mu / inv_sigma gradients (fixed order inside a block and across blocks)
constexpr int GBP_THREADS = 256;
constexpr int GBP_EDGES_PER_BLOCK = 2048;

__global__ void __launch_bounds__(GBP_THREADS)
k_gaussian_bp(i64 nnz, int K, int dim, const float* pseudo, const float* mu, const float* sig,
              const float* gg, float* pseudo_out, float* part /* [blocks][2][K*dim] */) {
  extern __shared__ float sm[];  // [GBP_THREADS/32][2*K*dim]
  const int kd = K * dim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const i64 e_begin = (i64)blockIdx.x * GBP_EDGES_PER_BLOCK;
  const i64 e_end = (e_begin + GBP_EDGES_PER_BLOCK < nnz) ? e_begin + GBP_EDGES_PER_BLOCK : nnz;
  // pseudo gradient: one thread per (edge, d)
  for (i64 t = e_begin * dim + threadIdx.x; t < e_end * dim; t += GBP_THREADS) {
    const i64 e = t / dim;
    const int d = (int)(t % dim);
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const float w = gauss_w(pseudo, mu, sig, e, k, dim) * __ldg(gg + e * K + k);
      const float s = __ldg(sig + k * dim + d);
      const float tt = (__ldg(pseudo + e * dim + d) - __ldg(mu + k * dim + d)) * s;
      acc = fmaf(-w * tt, s, acc);
    }
    pseudo_out[t] = acc;
  }
  // mu / sigma gradients: for each (k,d), threads stride over edges, then reduce
  for (int i = 0; i < kd; ++i) {
    const int k = i / dim, d = i % dim;
    const float s = __ldg(sig + i), m = __ldg(mu + i);
    float am = 0.f, as = 0.f;
    for (i64 e = e_begin + threadIdx.x; e < e_end; e += GBP_THREADS) {
      const float w = gauss_w(pseudo, mu, sig, e, k, dim) * __ldg(gg + e * K + k);
      const float diff = __ldg(pseudo + e * dim + d) - m;
      const float tt = diff * s;
      am = fmaf(w * tt, s, am);
      as = fmaf(-w * tt, diff, as);
    }
    for (int o = 16; o; o >>= 1) {
      am += __shfl_xor_sync(DGNN_FULL, am, o);
      as += __shfl_xor_sync(DGNN_FULL, as, o);
    }
    if (lane == 0) { sm[warp * 2 * kd + i] = am; sm[warp * 2 * kd + kd + i] = as; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * kd; i += GBP_THREADS) {
    float s = 0.f;
    for (int w = 0; w < GBP_THREADS / 32; ++w) s += sm[w * 2 * kd + i];
    part[(i64)blockIdx.x * 2 * kd + i] = s;
  }
}

__global__ void k_gaussian_bp_final(i64 blocks, int kd, const float* part, float* mu_out, float* sigma_out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * kd) return;
  float s = 0.f;
  for (i64 b = 0; b < blocks; ++b) s += part[b * 2 * kd + i];
  if (i < kd) mu_out[i] = s; else sigma_out[i - kd] = s;
}

inline i64 gbp_blocks(i64 nnz) { return (nnz + GBP_EDGES_PER_BLOCK - 1) / GBP_EDGES_PER_BLOCK; }

template <class Op>
int launch_sddmm_op(const FastShape& fs, i64 n_rows, i64 nnz, int h, const void* row_ptr, int idx_bits,
                    const int* col_ind, const float* a, const float* b, float* out, void* ws, cudaStream_t s) {
  Op op;
  op.ws = nullptr; op.slot_stride = 0; op.skip_empty = 1;
  op.n_rows = n_rows; op.nnz = nnz; op.indptr = row_ptr; op.idx_bits = idx_bits;
  op.H = h; op.hf4 = fs.hf4; op.f4_shift = fs.f4_shift; op.col_ind = col_ind;
  op.a = reinterpret_cast<const float4*>(a); op.b = reinterpret_cast<const float4*>(b); op.out = out;
  return dgnn_launch_trio(op, reinterpret_cast<unsigned long long*>(ws), s);
}

template <int VPL, int LPR, class... A>
int launch_sddmm(const FastShape& fs, A... args) {
  if constexpr (VPL > 1 && DGNN_LD256) {
    if (fs.same_head) return launch_sddmm_op<SddmmOpSH<VPL>>(fs, args...);
  }
  return launch_sddmm_op<SddmmOp<VPL, LPR>>(fs, args...);
}

template <int VPL, int LPR>
int launch_gmm(const FastShape& fs, i64 n_rows, i64 nnz, int K, int dim, int f, const void* row_ptr,
               int idx_bits, const int* col_ind, const float* feat, const float* pseudo, const float* mu,
               const float* sig, float* out, void* ws, cudaStream_t s) {
  GmmOp<VPL, LPR> op;
  op.n_rows = n_rows; op.nnz = nnz; op.indptr = row_ptr; op.idx_bits = idx_bits;
  op.H = K; op.hf4 = fs.hf4; op.f4_shift = fs.f4_shift; op.dim = dim; op.col_ind = col_ind;
  op.feat = reinterpret_cast<const float4*>(feat); op.pseudo = pseudo; op.mu = mu; op.sig = sig;
  op.out = reinterpret_cast<float4*>(out);
  op.ws = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + DGNN_WS_HEADER);
  op.slot_stride = (i64)K * f; op.skip_empty = 0;
  return dgnn_launch_trio(op, reinterpret_cast<unsigned long long*>(ws), s);
}

}  // namespace

extern "C" {

size_t dgnn_mhsddmm_workspace_bytes(void) { return DGNN_WS_HEADER; }

int dgnn_mhsddmm(int64_t n_rows, int64_t nnz, int h, int f, const void* row_ptr, int idx_bits,
                 const int32_t* col_ind, const float* a, const float* b, float* out, void* workspace,
                 size_t workspace_bytes, void* stream) {
  if (n_rows < 0 || nnz < 0 || h <= 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (idx_bits != 32 && idx_bits != 64) return DGNN_ERR_IDX_BITS;
  if (idx_bits == 32 && nnz > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (n_rows == 0 || nnz == 0) return DGNN_OK;
  if (!row_ptr || !col_ind || !a || !b || !out) return DGNN_ERR_NULL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FastShape fs = fast_shape(h, f);
  fs.same_head = fs.ok && fs.vpl > 1 && (1 << fs.f4_shift) >= fs.vpl &&
                 ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 31) == 0;
  if (fs.ok && aligned16(a) && aligned16(b)) {
    if (!workspace || workspace_bytes < DGNN_WS_HEADER) return DGNN_ERR_WORKSPACE;
#define SD_ARGS fs, n_rows, nnz, h, row_ptr, idx_bits, col_ind, a, b, out, workspace, s
    switch (fs.vpl) {
      case 1:
        if (fs.lpr == 8) return launch_sddmm<1, 8>(SD_ARGS);
        if (fs.lpr == 16) return launch_sddmm<1, 16>(SD_ARGS);
        return launch_sddmm<1, 32>(SD_ARGS);
      case 2: return launch_sddmm<2, 32>(SD_ARGS);
      case 4: return launch_sddmm<4, 32>(SD_ARGS);
      default: return launch_sddmm<8, 32>(SD_ARGS);
    }
#undef SD_ARGS
  }
  k_sddmm_generic<<<dgnn_grid(n_rows * h, DGNN_WARPS), DGNN_THREADS, 0, s>>>(n_rows, h, f, row_ptr, idx_bits,
                                                                           col_ind, a, b, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_coo_sddmm(int64_t nnz, int k, const int32_t* row_ind, const int32_t* col_ind, const float* d1,
                   const float* d2, float* out, void* stream) {
  if (nnz < 0 || k <= 0) return DGNN_ERR_SHAPE;
  if (nnz == 0) return DGNN_OK;
  if (!row_ind || !col_ind || !d1 || !d2 || !out) return DGNN_ERR_NULL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = dgnn_grid(nnz, DGNN_WARPS);
  if (k % 4 == 0 && aligned16(d1) && aligned16(d2))
    k_coo_sddmm<float4><<<grid, DGNN_THREADS, 0, s>>>(nnz, k / 4, row_ind, col_ind, reinterpret_cast<const float4*>(d1),
                                                     reinterpret_cast<const float4*>(d2), out);
  else
    k_coo_sddmm<float><<<grid, DGNN_THREADS, 0, s>>>(nnz, k, row_ind, col_ind, d1, d2, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_mhtranspose(int64_t nnz, int h, const int32_t* permute, const float* in, float* out, void* stream) {
  if (nnz < 0 || h <= 0) return DGNN_ERR_SHAPE;
  if (nnz == 0) return DGNN_OK;
  if (!permute || !in || !out) return DGNN_ERR_NULL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (h % 4 == 0 && aligned16(in) && aligned16(out)) {
    k_transpose4<<<dgnn_grid(nnz * (h / 4), 256), 256, 0, s>>>(nnz, h / 4, permute,
                                                             reinterpret_cast<const float4*>(in),
                                                             reinterpret_cast<float4*>(out));
  } else {
    k_transpose1<<<dgnn_grid(nnz * h, 256), 256, 0, s>>>(nnz, h, permute, in, out);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

size_t dgnn_gmm_forward_workspace_bytes(int64_t n_rows, int64_t nnz, int kernels, int f) {
  (void)n_rows;
  if (nnz <= DGNN_SEG || kernels <= 0 || f <= 0) return DGNN_WS_HEADER;
  return DGNN_WS_HEADER + up256((size_t)(2 * dgnn_num_chunks(nnz)) * kernels * f * sizeof(float));
}

int dgnn_gmm_forward(int64_t n_rows, int64_t nnz, int kernels, int dim, int f, const void* row_ptr,
                     int idx_bits, const int32_t* col_ind, const float* node_feat, const float* pseudo,
                     const float* mu, const float* inv_sigma, float* out, void* workspace,
                     size_t workspace_bytes, void* stream) {
  if (n_rows < 0 || nnz < 0 || kernels <= 0 || dim <= 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (idx_bits != 32 && idx_bits != 64) return DGNN_ERR_IDX_BITS;
  if (idx_bits == 32 && nnz > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (n_rows == 0) return DGNN_OK;
  if (!row_ptr || !out || !mu || !inv_sigma || (nnz > 0 && (!col_ind || !node_feat || !pseudo))) return DGNN_ERR_NULL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const FastShape fs = fast_shape(kernels, f);
  if (fs.ok && aligned16(node_feat) && aligned16(out)) {
    if (!workspace || workspace_bytes < dgnn_gmm_forward_workspace_bytes(n_rows, nnz, kernels, f))
      return DGNN_ERR_WORKSPACE;
    if (!aligned16(workspace)) return DGNN_ERR_ALIGN;
#define GM_ARGS fs, n_rows, nnz, kernels, dim, f, row_ptr, idx_bits, col_ind, node_feat, pseudo, mu, inv_sigma, out, workspace, s
    switch (fs.vpl) {
      case 1:
        if (fs.lpr == 8) return launch_gmm<1, 8>(GM_ARGS);
        if (fs.lpr == 16) return launch_gmm<1, 16>(GM_ARGS);
        return launch_gmm<1, 32>(GM_ARGS);
      case 2: return launch_gmm<2, 32>(GM_ARGS);
      case 4: return launch_gmm<4, 32>(GM_ARGS);
      default: return launch_gmm<8, 32>(GM_ARGS);
    }
#undef GM_ARGS
  }
  k_gmm_generic<<<dgnn_grid(n_rows * kernels, DGNN_WARPS), DGNN_THREADS, 0, s>>>(
      n_rows, kernels, dim, f, row_ptr, idx_bits, col_ind, node_feat, pseudo, mu, inv_sigma, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_gaussian(int64_t nnz, int kernels, int dim, const float* pseudo, const float* mu,
                  const float* inv_sigma, float* gauss, void* stream) {
  if (nnz < 0 || kernels <= 0 || dim <= 0) return DGNN_ERR_SHAPE;
  if (nnz == 0) return DGNN_OK;
  if (!pseudo || !mu || !inv_sigma || !gauss) return DGNN_ERR_NULL;
  k_gaussian<<<dgnn_grid(nnz * kernels, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      nnz, kernels, dim, pseudo, mu, inv_sigma, gauss);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

size_t dgnn_gaussian_bp_workspace_bytes(int64_t nnz, int kernels, int dim) {
  if (nnz <= 0 || kernels <= 0 || dim <= 0) return 256;
  return up256((size_t)gbp_blocks(nnz) * 2 * kernels * dim * sizeof(float)) + 256;
}

int dgnn_gaussian_bp(int64_t nnz, int kernels, int dim, const float* pseudo, const float* mu,
                     const float* inv_sigma, const float* grad_gauss, float* pseudo_out, float* mu_out,
                     float* sigma_out, void* workspace, size_t workspace_bytes, void* stream) {
  if (nnz < 0 || kernels <= 0 || dim <= 0) return DGNN_ERR_SHAPE;
  if (!mu || !inv_sigma || !mu_out || !sigma_out) return DGNN_ERR_NULL;
  const int kd = kernels * dim;
  const size_t smem = (size_t)(GBP_THREADS / 32) * 2 * kd * sizeof(float);
  if (smem > 48 * 1024) return DGNN_ERR_SHAPE;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const i64 blocks = nnz > 0 ? gbp_blocks(nnz) : 0;
  if (nnz > 0) {
    if (!pseudo || !grad_gauss || !pseudo_out) return DGNN_ERR_NULL;
    if (!workspace || workspace_bytes < dgnn_gaussian_bp_workspace_bytes(nnz, kernels, dim)) return DGNN_ERR_WORKSPACE;
    k_gaussian_bp<<<(unsigned)blocks, GBP_THREADS, smem, s>>>(nnz, kernels, dim, pseudo, mu, inv_sigma, grad_gauss,
                                                             pseudo_out, reinterpret_cast<float*>(workspace));
  }
  k_gaussian_bp_final<<<dgnn_grid(2 * kd, 128), 128, 0, s>>>(blocks, kd, reinterpret_cast<const float*>(workspace),
                                                           mu_out, sigma_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

}  // extern "C"

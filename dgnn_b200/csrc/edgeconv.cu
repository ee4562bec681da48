// EdgeConv max-aggregation over a regular kNN graph (k neighbours per point).
//
// Forward: one thread per (point, float4 of features); the k neighbour rows are
// gathered as contiguous F*4-byte rows (lanes of a point read consecutive
// 16-byte vectors), four neighbours in flight.  The reference instead lays its
// lanes over the neighbours and gathers one float per lane from k rows.
// Backward: zero fill, then a scatter-add of grad_out into the arg-max rows.
#include "common.cuh"

namespace {

template <typename V> struct VecOps;
template <> struct VecOps<float4> {
  static constexpr int W = 4;
  __device__ static float get(const float4& a, int i) { return i == 0 ? a.x : i == 1 ? a.y : i == 2 ? a.z : a.w; }
};
template <> struct VecOps<float> {
  static constexpr int W = 1;
  __device__ static float get(const float& a, int) { return a; }
};

template <typename V>
__global__ void __launch_bounds__(256)
k_edgeconv_fwd(i64 m, int fv /* vectors per row */, int k, const int* src_ind, const V* h_src,
               const V* h_dst, V* out, int* max_idx) {
  constexpr int W = VecOps<V>::W;
  constexpr int U = 4;
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= m * fv) return;
  const i64 i = t / fv;
  const int q = (int)(t % fv);
  const V a = __ldg(h_dst + t);
  float best[W];
  int bid[W];
#pragma unroll
  for (int c = 0; c < W; ++c) { best[c] = -INFINITY; bid[c] = -1; }
  const int* nb = src_ind + i * k;
  for (int j = 0; j < k; j += U) {
    int id[U];
    V x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      id[u] = (j + u < k) ? __ldg(nb + j + u) : 0;
      if (j + u < k) x[u] = __ldg(h_src + (i64)id[u] * fv + q);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (j + u < k) {
#pragma unroll
        for (int c = 0; c < W; ++c) {
          const float s = VecOps<V>::get(a, c) + VecOps<V>::get(x[u], c);
          if (s > best[c] || bid[c] < 0) { best[c] = s; bid[c] = id[u]; }
        }
      }
    }
  }
  if (W == 4) {
    reinterpret_cast<float4*>(out)[t] = make_float4(best[0], best[1 % W], best[2 % W], best[3 % W]);
    reinterpret_cast<int4*>(max_idx)[t] = make_int4(bid[0], bid[1 % W], bid[2 % W], bid[3 % W]);
  } else {
    reinterpret_cast<float*>(out)[t] = best[0];
    max_idx[t] = bid[0];
  }
}

__global__ void k_edgeconv_bwd(i64 total, int f, const int* max_idx, const float* grad_out, float* grad_src) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int id = __ldg(max_idx + t);
  if (id < 0) return;  // k == 0: no neighbour was selected
  atomicAdd(grad_src + (i64)id * f + (t % f), __ldg(grad_out + t));
}

// Reproducible backward: one thread per (source point s, feature j).  The in-edges of s come from the CSC form of the
// neighbour graph (destinations ascending); destination i contributes grad_out[i, j] when it selected s for feature j,
// added in ascending i.  A destination that lists s more than once (adjacent after the sort) is counted once, as in
// the forward, which keeps the first of equal sums.  No atomics: the sum has one fixed order.
__global__ void k_edgeconv_bwd_ordered(i64 m, int f, const int* col_ptr, const int* row_ind, const int* max_idx,
                                       const float* grad_out, float* grad_src) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= m * f) return;
  const i64 s = t / f;
  const int j = (int)(t - s * f);
  const int e0 = __ldg(col_ptr + s), e1 = __ldg(col_ptr + s + 1);
  float acc = 0.f;
  int prev = -1;
  for (int e = e0; e < e1; ++e) {
    const int i = __ldg(row_ind + e);
    if (i == prev) continue;
    prev = i;
    if (__ldg(max_idx + (i64)i * f + j) == (int)s) acc += __ldg(grad_out + (i64)i * f + j);
  }
  grad_src[t] = acc;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" {

int dgnn_edgeconv_forward(int64_t m, int f, int k, const int32_t* src_ind, const float* h_src,
                          const float* h_dst, float* out, int32_t* max_idx, void* stream) {
  if (m < 0 || f <= 0 || k < 0) return DGNN_ERR_SHAPE;
  if (m > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (m == 0) return DGNN_OK;
  if (!h_src || !h_dst || !out || !max_idx || (k > 0 && !src_ind)) return DGNN_ERR_NULL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (f % 4 == 0 && aligned16(h_src) && aligned16(h_dst) && aligned16(out) && aligned16(max_idx)) {
    k_edgeconv_fwd<float4><<<dgnn_grid(m * (f / 4), 256), 256, 0, s>>>(
        m, f / 4, k, src_ind, reinterpret_cast<const float4*>(h_src), reinterpret_cast<const float4*>(h_dst),
        reinterpret_cast<float4*>(out), max_idx);
  } else {
    k_edgeconv_fwd<float><<<dgnn_grid(m * f, 256), 256, 0, s>>>(m, f, k, src_ind, h_src, h_dst, out, max_idx);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_edgeconv_backward(int64_t m, int f, const int32_t* max_idx, const float* grad_out,
                           float* grad_src, void* stream) {
  if (m < 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (m == 0) return DGNN_OK;
  if (!max_idx || !grad_out || !grad_src) return DGNN_ERR_NULL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(grad_src, 0, (size_t)m * f * sizeof(float), s);
  if (e != cudaSuccess) return (int)e;
  k_edgeconv_bwd<<<dgnn_grid(m * f, 256), 256, 0, s>>>(m * f, f, max_idx, grad_out, grad_src);
  e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_edgeconv_backward_ordered(int64_t m, int f, const int32_t* col_ptr, const int32_t* row_ind,
                                   const int32_t* max_idx, const float* grad_out, float* grad_src, void* stream) {
  if (m < 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (m > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (m == 0) return DGNN_OK;
  if (!col_ptr || !max_idx || !grad_out || !grad_src) return DGNN_ERR_NULL;   // row_ind may be NULL for a graph without edges
  k_edgeconv_bwd_ordered<<<dgnn_grid(m * f, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      m, f, col_ptr, row_ind, max_idx, grad_out, grad_src);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

}  // extern "C"

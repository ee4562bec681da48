// k nearest neighbours inside every cloud of a batch of point clouds (the graph EdgeConv runs on).
//
// One thread per query point.  The candidates of the cloud pass through shared memory in tiles (all
// threads of a CTA read the same candidate at the same time: a broadcast), the query's own coordinates sit
// in a padded shared-memory row, and every thread keeps its k best (squared distance, index) pairs sorted
// in registers: a candidate is compared with the current worst first, so almost all of them cost one
// comparison, and the few that enter ripple down an unrolled compare-exchange chain.
// Squared distances are accumulated dimension by dimension with separately rounded multiply and add (no
// fused multiply-add), candidates are visited in index order and a candidate only displaces strictly
// larger distances: the result is the stable sort of the distances -- ties go to the smaller index, the
// point itself (distance 0) comes first -- reproducible bit for bit on any device or on a CPU.
#include "common.cuh"

namespace {

constexpr int KNN_THREADS = 128;
constexpr int KNN_TILE = 256;   // candidates per shared-memory tile

template <int KCAP>
__global__ void __launch_bounds__(KNN_THREADS)
k_knn(int n_points, int dim, int k, const float* __restrict__ pts, int* __restrict__ out) {
  extern __shared__ float knn_sm[];
  const int dpad = dim | 1;                         // odd row length: threads reading their own row hit different banks
  float* qrow = knn_sm;                             // [KNN_THREADS][dpad]
  float* cand = knn_sm + KNN_THREADS * dpad;        // [KNN_TILE][dim]
  const i64 cloud = blockIdx.y;
  const float* base = pts + cloud * (i64)n_points * dim;
  const int q = blockIdx.x * KNN_THREADS + threadIdx.x;
  const bool live = q < n_points;
  for (int d = 0; d < dim; ++d) qrow[threadIdx.x * dpad + d] = live ? base[(i64)q * dim + d] : 0.f;
  float best_d[KCAP];
  int best_i[KCAP];
#pragma unroll
  for (int j = 0; j < KCAP; ++j) { best_d[j] = __int_as_float(0x7f800000); best_i[j] = -1; }
  float worst = __int_as_float(0x7f800000);         // distance at list position k-1
  for (int t0 = 0; t0 < n_points; t0 += KNN_TILE) {
    const int cnt = n_points - t0 < KNN_TILE ? n_points - t0 : KNN_TILE;
    __syncthreads();
    for (int i = threadIdx.x; i < cnt * dim; i += KNN_THREADS) cand[i] = base[(i64)t0 * dim + i];
    __syncthreads();
    for (int c = 0; c < cnt; ++c) {
      float d2 = 0.f;
      for (int d = 0; d < dim; ++d) {
        const float diff = __fsub_rn(qrow[threadIdx.x * dpad + d], cand[c * dim + d]);
        d2 = __fadd_rn(d2, __fmul_rn(diff, diff));
      }
      if (d2 < worst) {                             // enters the list: behind every entry that is <= d2
        float cd = d2;
        int ci = t0 + c;
        bool placed = false;                        // once placed, every later entry moves down one position
#pragma unroll
        for (int j = 0; j < KCAP; ++j) {
          if (j < k && (placed || cd < best_d[j])) {
            placed = true;
            const float td = best_d[j]; best_d[j] = cd; cd = td;
            const int ti = best_i[j]; best_i[j] = ci; ci = ti;
          }
        }
#pragma unroll
        for (int j = 0; j < KCAP; ++j) if (j == k - 1) worst = best_d[j];
      }
    }
  }
  if (!live) return;
  int* dst = out + (cloud * n_points + q) * (i64)k;
#pragma unroll
  for (int j = 0; j < KCAP; ++j)
    if (j < k) dst[j] = (int)(cloud * n_points) + best_i[j];
}

}  // namespace

extern "C" {

int dgnn_knn_max_k(void) { return 32; }

int dgnn_knn_graph(int64_t n_clouds, int64_t n_points, int dim, int k, const float* points, int32_t* src_ind, void* stream) {
  if (n_clouds < 0 || n_points < 0 || dim <= 0 || k <= 0) return DGNN_ERR_SHAPE;
  if (k > 32 || k > n_points) return DGNN_ERR_VALUE;
  if (n_clouds * n_points > 0x7fffffffLL || n_clouds > 65535) return DGNN_ERR_OVERFLOW;
  if (n_clouds == 0 || n_points == 0) return DGNN_OK;
  if (!points || !src_ind) return DGNN_ERR_NULL;
  const size_t smem = ((size_t)KNN_THREADS * (dim | 1) + (size_t)KNN_TILE * dim) * sizeof(float);
  if (smem > 200 * 1024) return DGNN_ERR_SHAPE;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)((n_points + KNN_THREADS - 1) / KNN_THREADS), (unsigned)n_clouds);
  cudaError_t e;
  if (k <= 8) {
    if ((e = dgnn_allow_smem(k_knn<8>, smem)) != cudaSuccess) return (int)e;
    k_knn<8><<<grid, KNN_THREADS, smem, s>>>((int)n_points, dim, k, points, src_ind);
  } else if (k <= 16) {
    if ((e = dgnn_allow_smem(k_knn<16>, smem)) != cudaSuccess) return (int)e;
    k_knn<16><<<grid, KNN_THREADS, smem, s>>>((int)n_points, dim, k, points, src_ind);
  } else {
    if ((e = dgnn_allow_smem(k_knn<32>, smem)) != cudaSuccess) return (int)e;
    k_knn<32><<<grid, KNN_THREADS, smem, s>>>((int)n_points, dim, k, points, src_ind);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

}  // extern "C"

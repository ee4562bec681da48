// Which rows of a gathered tensor should stay in the L2.
//
// The fused GAT sweeps gather one feature row per edge out of a tensor that is far larger than the 126 MB L2
// (2.46 GB at 2.4 M nodes x 8 heads x 32).  On a power-law graph a few rows receive most of the references:
// at R-MAT 2.4 M / 120 M the 60,000 most referenced rows (61 MB) take 64 % of all gathers, the 100,000 most
// referenced 74 %.  The L2's own replacement keeps them only as long as no burst of once-read rows pushes them
// out -- the measured hit rate of the forward sweep is 48 %.  dgnn_hot_rows marks the rows whose reference
// count (the length of their CSR / CSC segment) is at least the smallest threshold that selects no more than
// `max_hot` rows, one bit per row; the sweeps load marked rows with the L2 evict_last priority and everything
// else normally, and write their results with streaming stores.
//
// Three small launches over the index pointer: a histogram of the segment lengths (clamped to HOT_BINS - 1), a
// one-CTA suffix scan that finds the threshold, and a ballot pass that writes the bit words.
#include "common.cuh"

namespace {

constexpr int HOT_BINS = 4096;
constexpr int HOT_THREADS = 256;

__global__ void __launch_bounds__(HOT_THREADS)
k_hot_hist(i64 n, const void* indptr, int bits, unsigned* hist) {
  __shared__ unsigned sh[HOT_BINS];
  for (int i = threadIdx.x; i < HOT_BINS; i += HOT_THREADS) sh[i] = 0;
  __syncthreads();
  for (i64 r = (i64)blockIdx.x * HOT_THREADS + threadIdx.x; r < n; r += (i64)gridDim.x * HOT_THREADS) {
    const i64 d = ldp(indptr, bits, r + 1) - ldp(indptr, bits, r);
    if (d > 0) atomicAdd(&sh[d < HOT_BINS ? (int)d : HOT_BINS - 1], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < HOT_BINS; i += HOT_THREADS)
    if (sh[i]) atomicAdd(hist + i, sh[i]);
}

// threshold = smallest t >= 1 with #{rows: length >= t} <= max_hot (HOT_BINS if even the last bin is too full)
__global__ void __launch_bounds__(1024)
k_hot_threshold(const unsigned* hist, i64 max_hot, unsigned* thr) {
  __shared__ unsigned long long suf[HOT_BINS + 1];   // suf[t] = rows of length >= t
  __shared__ unsigned long long part[1024];
  constexpr int PER = HOT_BINS / 1024;
  const int t0 = threadIdx.x * PER;
  unsigned long long own = 0;
  for (int j = 0; j < PER; ++j) own += hist[t0 + j];
  part[threadIdx.x] = own;
  __syncthreads();
  if (threadIdx.x == 0) {                            // 1024 additions, from the top
    unsigned long long run = 0;
    for (int i = 1023; i >= 0; --i) { const unsigned long long v = part[i]; part[i] = run; run += v; }
  }
  __syncthreads();
  unsigned long long run = part[threadIdx.x];        // rows in the bins above this thread's
  for (int j = PER - 1; j >= 0; --j) { run += hist[t0 + j]; suf[t0 + j] = run; }
  if (threadIdx.x == 0) { suf[HOT_BINS] = 0; *thr = HOT_BINS; }
  __syncthreads();
  // suf is non-increasing in t: the threshold is the one t with suf[t] <= max_hot < suf[t-1]
  for (int j = 0; j < PER; ++j) {
    const int t = t0 + j;
    if (t >= 1 && suf[t] <= (unsigned long long)max_hot && (t == 1 || suf[t - 1] > (unsigned long long)max_hot)) *thr = (unsigned)t;
  }
}

__global__ void __launch_bounds__(HOT_THREADS)
k_hot_bits(i64 n, const void* indptr, int bits, const unsigned* thr, unsigned* out) {
  const i64 r = (i64)blockIdx.x * HOT_THREADS + threadIdx.x;   // a warp covers 32 consecutive rows = one word
  const i64 t = (i64)__ldg(thr);
  bool hot = false;
  if (r < n) hot = ldp(indptr, bits, r + 1) - ldp(indptr, bits, r) >= t;
  const unsigned w = __ballot_sync(DGNN_FULL, hot);
  if ((threadIdx.x & 31) == 0 && r < n) out[r >> 5] = w;
}

}  // namespace

extern "C" {

// Part of the L2 set aside for lines loaded with the evict_last priority (a limit of the calling process's CUDA
// context; it ends with the process).  Returns the size in force afterwards, or a negative CUDA error.
int64_t dgnn_l2_set_aside(int64_t bytes) {
  if (bytes < 0) return -(int64_t)cudaErrorInvalidValue;
  int dev = 0, max_bytes = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&max_bytes, cudaDevAttrMaxPersistingL2CacheSize, dev);
  if (e != cudaSuccess) return -(int64_t)e;
  if (bytes > max_bytes) bytes = max_bytes;
  e = cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, (size_t)bytes);
  if (e != cudaSuccess) return -(int64_t)e;
  size_t now = 0;
  e = cudaDeviceGetLimit(&now, cudaLimitPersistingL2CacheSize);
  return e == cudaSuccess ? (int64_t)now : -(int64_t)e;
}

size_t dgnn_hot_rows_workspace_bytes(void) { return (HOT_BINS + 4) * sizeof(unsigned); }

int dgnn_hot_rows(int64_t n, const void* indptr, int idx_bits, int64_t max_hot, uint32_t* hot_bits,
                  void* workspace, size_t workspace_bytes, void* stream) {
  if (n < 0 || max_hot < 0 || (idx_bits != 32 && idx_bits != 64)) return DGNN_ERR_SHAPE;
  if (n == 0) return DGNN_OK;
  if (!indptr || !hot_bits) return DGNN_ERR_NULL;
  if (!workspace || workspace_bytes < dgnn_hot_rows_workspace_bytes()) return DGNN_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 3) return DGNN_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  unsigned* hist = reinterpret_cast<unsigned*>(workspace);
  unsigned* thr = hist + HOT_BINS;
  cudaError_t e = cudaMemsetAsync(workspace, 0, dgnn_hot_rows_workspace_bytes(), s);
  if (e != cudaSuccess) return (int)e;
  i64 ctas = (n + HOT_THREADS - 1) / HOT_THREADS;
  if (ctas > 148 * 8) ctas = 148 * 8;
  k_hot_hist<<<(unsigned)ctas, HOT_THREADS, 0, s>>>(n, indptr, idx_bits, hist);
  k_hot_threshold<<<1, 1024, 0, s>>>(hist, max_hot, thr);
  k_hot_bits<<<(unsigned)((n + HOT_THREADS - 1) / HOT_THREADS), HOT_THREADS, 0, s>>>(n, indptr, idx_bits, thr, hot_bits);
  e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

}  // extern "C"

// Status strings, version and the counter-based uniform generator.
#include "common.cuh"

namespace {

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11)
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__global__ void k_uniform(uint64_t seed, uint64_t offset, i64 n, float* out) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;  // one counter -> 4 floats
  if (t * 4 >= n) return;
  const uint64_t ctr = offset + (uint64_t)t;
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const i64 p = t * 4 + i;
    if (p < n) out[p] = ((float)(c[i] >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
  }
}

// ---- guard mode: validation of the index arrays a caller hands over ------------------------------------
// report[0] = first kind of defect seen (0 none; 1 ptr[0] != 0; 2 ptr decreases; 3 ptr[n] != nnz; 4 index out of
// range), report[1] = smallest position at which a defect of any kind was seen (atomicMin), report[2] = its value
__device__ __forceinline__ void guard_note(int* report, int kind, i64 pos, i64 value) {
  atomicCAS(report, 0, kind);
  const int p = pos > 0x7fffffffLL ? 0x7fffffff : (int)pos;
  if (atomicMin(report + 1, p) > p) report[2] = (int)value;
}

__global__ void k_check_ptr(i64 n, i64 nnz, const void* ptr, int bits, int* report) {
  const i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  const i64 v = ldp(ptr, bits, i);
  if (i == 0 && v != 0) guard_note(report, 1, 0, v);
  if (i == n && v != nnz) guard_note(report, 3, n, v);
  if (i < n && ldp(ptr, bits, i + 1) < v) guard_note(report, 2, i, v);
}

__global__ void k_check_index(i64 n, const int* idx, i64 limit, int* report) {
  const i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int v = __ldg(idx + i);
  if (v < 0 || (i64)v >= limit) guard_note(report, 4, i, v);
}

}  // namespace

extern "C" {

int dgnn_version(void) { return 110; }

int dgnn_check_ptr(int64_t n, int64_t nnz, const void* ptr, int idx_bits, int32_t* report, void* stream) {
  if (n < 0 || nnz < 0) return DGNN_ERR_SHAPE;
  if (idx_bits != 32 && idx_bits != 64) return DGNN_ERR_IDX_BITS;
  if (!ptr || !report) return DGNN_ERR_NULL;
  k_check_ptr<<<dgnn_grid(n + 1, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(n, nnz, ptr, idx_bits, report);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_check_index(int64_t n, const int32_t* idx, int64_t limit, int32_t* report, void* stream) {
  if (n < 0 || limit < 0) return DGNN_ERR_SHAPE;
  if (n == 0) return DGNN_OK;
  if (!idx || !report) return DGNN_ERR_NULL;
  k_check_index<<<dgnn_grid(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(n, idx, limit, report);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int64_t dgnn_seg_chunk(void) { return DGNN_SEG; }

const char* dgnn_status_string(int status) {
  switch (status) {
    case DGNN_OK: return "ok";
    case DGNN_ERR_NULL: return "a required pointer is NULL";
    case DGNN_ERR_SHAPE: return "negative or inconsistent size";
    case DGNN_ERR_IDX_BITS: return "idx_bits must be 32 or 64";
    case DGNN_ERR_ALIGN: return "pointer is not 16-byte aligned";
    case DGNN_ERR_OVERFLOW: return "size does not fit the index type";
    case DGNN_ERR_WORKSPACE: return "workspace missing or too small";
    case DGNN_ERR_VALUE: return "scalar argument out of range";
    case DGNN_ERR_STATIC_LIMIT: return "size exceeds the fixed scratch of the allocation-free entry point";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown dgnn status";
}

int dgnn_uniform_fill(uint64_t seed, uint64_t offset, int64_t n, float* out, void* stream) {
  if (n < 0) return DGNN_ERR_SHAPE;
  if (n == 0) return DGNN_OK;
  if (!out) return DGNN_ERR_NULL;
  const i64 ctrs = (n + 3) / 4;
  k_uniform<<<dgnn_grid(ctrs, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(seed, offset, n, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

}  // extern "C"

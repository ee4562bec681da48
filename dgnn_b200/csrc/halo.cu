// Halo exchange of the row-block sharded GAT layer, and the per-edge dropout randoms that go with it.
//
// A rank owns a block of nodes.  Its edges reference rows (source features and attention terms in the
// forward, grad_out and row statistics in the backward) of nodes that other ranks own; only the
// DISTINCT referenced rows are fetched, once per pass, into a local buffer laid out as
// [own rows | halo rows], and the graph arrays of the rank index that buffer.  k_halo_pull is the
// fetch: every halo row i is described by one code = (owner rank << 27) | row inside the owner's
// block, and the kernel copies that row out of the owner's buffer -- a pointer into this GPU's own
// memory or a peer mapping of another GPU's memory over NVLink (plain 16-byte loads; no TMA, no
// multicast).  Two tensors with the same row list (features + attention terms, or grad_out + row
// statistics) travel in one launch.  The grid is kept small so that the fetch runs beside the
// aggregation kernels of the rows that are already there.
#include "common.cuh"

namespace {

constexpr int HALO_MAX_RANKS = 16;
constexpr int HALO_SHIFT = 27;
constexpr int HALO_THREADS = 256;
constexpr int HALO_UNROLL = 4;

struct HaloPtrs {
  const float4* p[HALO_MAX_RANKS];
};

__device__ __forceinline__ float4 ld_stream(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// One tensor: dst[i, :] = src[rank_i][idx_i, :], rows of `vpr` float4 vectors.  A group of G = min(32, next power
// of two >= vpr) lanes owns a row (a whole warp for rows of 512 bytes or more, several rows per warp for short
// ones), so the row's code is read once per group and no division by the row length is needed; every group
// works on HALO_UNROLL rows at a time with all their loads issued before the first store.
__device__ __forceinline__ void pull_tensor(i64 n_rows, const int* codes, int n_ranks, i64 src_rows, const HaloPtrs& src,
                                            float4* dst, int vpr, int* status) {
  int g = 1;
  while (g < vpr && g < 32) g <<= 1;
  const int lane = threadIdx.x & 31;
  const int sub = lane & (g - 1);                        // lane inside its group
  const i64 groups_per_cta = (HALO_THREADS / 32) * (32 / g);
  const i64 group = (i64)blockIdx.x * groups_per_cta + (threadIdx.x >> 5) * (32 / g) + lane / g;
  const i64 step = (i64)gridDim.x * groups_per_cta;
  for (i64 row0 = group; row0 < n_rows; row0 += step * HALO_UNROLL) {
    const float4* from[HALO_UNROLL];
#pragma unroll
    for (int k = 0; k < HALO_UNROLL; ++k) {
      const i64 row = row0 + (i64)k * step;
      from[k] = nullptr;
      if (row < n_rows) {
        const unsigned code = (unsigned)__ldg(codes + row);
        const int rk = (int)(code >> HALO_SHIFT);
        const i64 idx = (i64)(code & ((1u << HALO_SHIFT) - 1));
        if (rk >= n_ranks || idx >= src_rows) {          // never dereference an address outside an owner's block
          if (status && sub == 0) atomicMax(status, 1);
        } else {
          from[k] = src.p[rk] + idx * vpr;
        }
      }
    }
    for (int q = sub; q < vpr; q += g) {
      float4 v[HALO_UNROLL];
#pragma unroll
      for (int k = 0; k < HALO_UNROLL; ++k)
        if (from[k]) v[k] = ld_stream(from[k] + q);
#pragma unroll
      for (int k = 0; k < HALO_UNROLL; ++k)
        if (from[k]) dst[(row0 + (i64)k * step) * vpr + q] = v[k];
    }
  }
}

__global__ void __launch_bounds__(HALO_THREADS)
k_halo_pull(i64 n_rows, const int* codes, int n_ranks, i64 src_rows, HaloPtrs src_a, float4* dst_a, int vpr_a,
            HaloPtrs src_b, float4* dst_b, int vpr_b, int* status) {
  pull_tensor(n_rows, codes, n_ranks, src_rows, src_a, dst_a, vpr_a, status);
  if (vpr_b > 0) pull_tensor(n_rows, codes, n_ranks, src_rows, src_b, dst_b, vpr_b, status);
}

// Philox4x32-10, the same stream as dgnn_uniform_fill: element e of the stream is word e % 4 of counter e / 4
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__global__ void k_uniform_edges(uint64_t seed, uint64_t offset, i64 nnz, int h, const int* edge_id, float* out) {
  const i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nnz * h) return;
  const i64 i = t / h;
  const uint64_t e = (uint64_t)__ldg(edge_id + i) * (uint64_t)h + (uint64_t)(t - i * h);
  const uint64_t ctr = offset + (e >> 2);
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  const uint32_t w = c[e & 3];
  out[t] = ((float)(w >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
}

}  // namespace

extern "C" {

int dgnn_halo_max_ranks(void) { return HALO_MAX_RANKS; }
int dgnn_halo_rank_shift(void) { return HALO_SHIFT; }

int dgnn_halo_pull(int64_t n_rows, const int32_t* codes, int n_ranks, int64_t src_rows,
                   const void* const* src_a, void* dst_a, int row_bytes_a,
                   const void* const* src_b, void* dst_b, int row_bytes_b,
                   int max_ctas, int32_t* status, void* stream) {
  if (n_rows < 0 || src_rows < 0 || n_ranks <= 0 || n_ranks > HALO_MAX_RANKS) return DGNN_ERR_SHAPE;
  if (src_rows > (1LL << HALO_SHIFT)) return DGNN_ERR_OVERFLOW;
  if (row_bytes_a <= 0 || row_bytes_a % 16 || row_bytes_b < 0 || row_bytes_b % 16) return DGNN_ERR_SHAPE;
  if (n_rows == 0) return DGNN_OK;
  if (!codes || !src_a || !dst_a || (row_bytes_b > 0 && (!src_b || !dst_b))) return DGNN_ERR_NULL;
  HaloPtrs a, b;
  for (int r = 0; r < HALO_MAX_RANKS; ++r) {
    a.p[r] = r < n_ranks ? reinterpret_cast<const float4*>(src_a[r]) : nullptr;
    b.p[r] = (r < n_ranks && row_bytes_b > 0) ? reinterpret_cast<const float4*>(src_b[r]) : nullptr;
    if (r < n_ranks && (!a.p[r] || (reinterpret_cast<uintptr_t>(a.p[r]) & 15))) return a.p[r] ? DGNN_ERR_ALIGN : DGNN_ERR_NULL;
    if (r < n_ranks && row_bytes_b > 0 && (!b.p[r] || (reinterpret_cast<uintptr_t>(b.p[r]) & 15)))
      return b.p[r] ? DGNN_ERR_ALIGN : DGNN_ERR_NULL;
  }
  if ((reinterpret_cast<uintptr_t>(dst_a) & 15) || (reinterpret_cast<uintptr_t>(dst_b) & 15)) return DGNN_ERR_ALIGN;
  const int vpr_a = row_bytes_a / 16, vpr_b = row_bytes_b / 16;
  // one warp (or part of one) per row of the wider tensor, HALO_UNROLL rows per group and step
  const int wide = vpr_a > vpr_b ? vpr_a : vpr_b;
  const i64 groups_per_cta = (HALO_THREADS / 32) * (wide >= 32 ? 1 : 32 / (wide <= 1 ? 1 : wide <= 2 ? 2 : wide <= 4 ? 4 : wide <= 8 ? 8 : wide <= 16 ? 16 : 32));
  i64 ctas = (n_rows + groups_per_cta * HALO_UNROLL - 1) / (groups_per_cta * HALO_UNROLL);
  if (max_ctas > 0 && ctas > max_ctas) ctas = max_ctas;
  if (ctas < 1) ctas = 1;
  k_halo_pull<<<(unsigned)ctas, HALO_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      n_rows, codes, n_ranks, src_rows, a, reinterpret_cast<float4*>(dst_a), vpr_a, b, reinterpret_cast<float4*>(dst_b),
      vpr_b, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int dgnn_uniform_fill_edges(uint64_t seed, uint64_t offset, int64_t nnz, int h, const int32_t* edge_id, float* out,
                            void* stream) {
  if (nnz < 0 || h <= 0) return DGNN_ERR_SHAPE;
  if (nnz == 0) return DGNN_OK;
  if (!edge_id || !out) return DGNN_ERR_NULL;
  k_uniform_edges<<<dgnn_grid(nnz * h, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(seed, offset, nnz, h,
                                                                                               edge_id, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

}  // extern "C"

// CSR -> CSC conversion and COO -> CSR for sm_100a, bit-exact and deterministic.
//
// csr2csc is a stable least-significant-digit radix sort of the CSR entries by
// column id (8-bit digits over ceil(log2(n_cols)) bits), carrying the CSR
// position (-> permute) and the row id (-> row_ind) as payload.  Each pass is
// histogram per tile -> exclusive scan over (digit, tile) -> stable scatter;
// ranks inside a tile come from warp match_any votes taken in index order, so
// entries of one column keep their CSR order exactly as the reference's
// cuSPARSE conversion (and scipy's tocsc) produce.  The last pass also writes
// the sorted column ids, and col_ptr[c] is the first position whose id is >= c
// (a binary search per column: no per-column histogram, no global atomics).
// Only shared-memory integer atomics (commutative) are used.
#include "common.cuh"
#include <mutex>

namespace {

constexpr int RS_TILE = 4096;                    // items per tile
constexpr int RADIX = 256;
constexpr int HIST_THREADS = RADIX;              // histogram kernel: one counter per thread
constexpr int HIST_IPT = RS_TILE / HIST_THREADS;
constexpr int RS_THREADS = 512;                  // scatter kernel
constexpr int RS_IPT = RS_TILE / RS_THREADS;     // 8 items per thread
constexpr int RS_WARPS = RS_THREADS / 32;
constexpr int RS_WARP_ITEMS = 32 * RS_IPT;       // consecutive items owned by one warp

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_IPT = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_IPT;  // 2048

inline size_t up256(size_t x) { return (x + 255) & ~size_t(255); }
inline i64 cdiv(i64 a, i64 b) { return (a + b - 1) / b; }

// ---- exclusive scan of unsigned ints (three-phase, recursive on the host) ----
__device__ __forceinline__ unsigned block_exclusive_scan(unsigned v, unsigned* total, unsigned* sm /*[32]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned inc = v;
  for (int o = 1; o < 32; o <<= 1) {
    unsigned t = __shfl_up_sync(DGNN_FULL, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) sm[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    unsigned w = lane < (int)(blockDim.x >> 5) ? sm[lane] : 0u;
    unsigned winc = w;
    for (int o = 1; o < 32; o <<= 1) {
      unsigned t = __shfl_up_sync(DGNN_FULL, winc, o);
      if (lane >= o) winc += t;
    }
    sm[lane] = winc - w;  // exclusive warp offsets
    if (lane == 31) *total = winc;
  }
  __syncthreads();
  const unsigned r = sm[warp] + inc - v;
  __syncthreads();
  return r;
}

// data[i] <- exclusive scan inside its tile; sums[tile] <- tile total
__global__ void __launch_bounds__(SCAN_THREADS)
k_scan_tiles(unsigned* data, i64 n, unsigned* sums) {
  __shared__ unsigned sm[32];
  __shared__ unsigned total;
  const i64 base = (i64)blockIdx.x * SCAN_TILE + (i64)threadIdx.x * SCAN_IPT;
  unsigned v[SCAN_IPT];
  unsigned s = 0;
#pragma unroll
  for (int i = 0; i < SCAN_IPT; ++i) {
    v[i] = (base + i < n) ? data[base + i] : 0u;
    s += v[i];
  }
  unsigned off = block_exclusive_scan(s, &total, sm);
#pragma unroll
  for (int i = 0; i < SCAN_IPT; ++i) {
    if (base + i < n) data[base + i] = off;
    off += v[i];
  }
  if (threadIdx.x == 0 && sums) sums[blockIdx.x] = total;
}

__global__ void k_scan_add(unsigned* data, i64 n, const unsigned* sums) {
  const i64 i = (i64)blockIdx.x * SCAN_TILE + threadIdx.x;
  const unsigned add = sums[blockIdx.x];
#pragma unroll
  for (int j = 0; j < SCAN_IPT; ++j) {
    const i64 p = i + (i64)j * SCAN_THREADS;
    if (p < n) data[p] += add;
  }
}

// number of scratch uints the recursive scan of n items needs
inline i64 scan_scratch_items(i64 n) {
  i64 total = 0;
  while (n > SCAN_TILE) {
    n = cdiv(n, SCAN_TILE);
    total += up256((size_t)n * 4) / 4;
  }
  return total + 64;
}

// in-place exclusive scan of data[0..n); scratch as sized above
int exclusive_scan(unsigned* data, i64 n, unsigned* scratch, cudaStream_t s) {
  if (n <= 0) return DGNN_OK;
  const i64 tiles = cdiv(n, SCAN_TILE);
  if (tiles == 1) {
    k_scan_tiles<<<1, SCAN_THREADS, 0, s>>>(data, n, nullptr);
    return DGNN_OK;
  }
  unsigned* sums = scratch;
  unsigned* next = scratch + up256((size_t)tiles * 4) / 4;
  k_scan_tiles<<<(unsigned)tiles, SCAN_THREADS, 0, s>>>(data, n, sums);
  int rc = exclusive_scan(sums, tiles, next, s);
  if (rc) return rc;
  k_scan_add<<<(unsigned)tiles, SCAN_THREADS, 0, s>>>(data, n, sums);
  return DGNN_OK;
}

// ---- col_ptr from the sorted column ids -------------------------------------
__global__ void k_col_ptr(i64 n_cols, i64 nnz, const unsigned* sorted_keys, void* out, int bits) {
  const i64 c = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (c > n_cols) return;
  i64 lo = 0, hi = nnz;  // first position whose column id is >= c
  while (lo < hi) {
    const i64 mid = (lo + hi) >> 1;
    if ((i64)__ldg(sorted_keys + mid) < c) lo = mid + 1; else hi = mid;
  }
  if (bits == 64) reinterpret_cast<i64*>(out)[c] = lo;
  else reinterpret_cast<int*>(out)[c] = (int)lo;
}

// row of the first entry of every run of RS_WARP_ITEMS consecutive CSR positions (the items one warp of the
// first pass owns): the warps then look their rows up between two neighbouring entries of this table
// instead of searching the whole index pointer
__global__ void k_warp_rows(i64 nnz, i64 n_rows, const void* row_ptr, int idx_bits, int* wrow, int items) {
  const i64 w = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  const i64 pos = w * items;
  if (pos < nnz) wrow[w] = (int)find_row(row_ptr, idx_bits, n_rows, pos);
}

// ---- radix passes -----------------------------------------------------------
// tile_hist layout: [digit][tile]
__global__ void __launch_bounds__(HIST_THREADS)
k_radix_hist(const unsigned* keys, i64 n, int shift, unsigned* tile_hist, i64 ntiles) {
  __shared__ unsigned h[RADIX];
  h[threadIdx.x] = 0;
  __syncthreads();
  const i64 base = (i64)blockIdx.x * RS_TILE;
#pragma unroll
  for (int i = 0; i < HIST_IPT; ++i) {
    const i64 idx = base + (i64)i * HIST_THREADS + threadIdx.x;
    if (idx < n) atomicAdd(&h[(__ldg(keys + idx) >> shift) & (RADIX - 1)], 1u);
  }
  __syncthreads();
  tile_hist[(i64)threadIdx.x * ntiles + blockIdx.x] = h[threadIdx.x];
}

// One tile of a stable pass.  (1) Every warp ranks its 256 consecutive items by
// digit with match_any votes taken in index order.  (2) The per-warp digit counts
// are turned into the position of every item inside the tile sorted by digit, and
// keys and payload are put in that order through shared memory.  (3) The sorted
// tile is written out: items of one digit are neighbours both in the tile and in
// the output, so a warp's store covers a few runs of consecutive addresses instead
// of 32 scattered words.
// FIRST: keys are the CSR column ids, payload (position,row) is generated here.
// TWO: a second payload (the row id) travels with the first; a plain (key, value) sort carries one.
template <bool FIRST, bool TWO>
__global__ void __launch_bounds__(RS_THREADS, 2)
k_radix_scatter(const unsigned* __restrict__ keys_in, const int* __restrict__ pos_in, const int* __restrict__ row_in,
                unsigned* __restrict__ keys_out, int* __restrict__ pos_out, int* __restrict__ row_out, i64 n, int shift,
                const unsigned* __restrict__ tile_off, i64 ntiles, const void* __restrict__ row_ptr, int idx_bits,
                i64 n_rows, const int* __restrict__ wrow) {
  __shared__ unsigned cnt[RS_WARPS][RADIX];  // per-warp digit counts, then per-warp start inside the sorted tile
  __shared__ unsigned gbase[RADIX];          // start of the digit's run in the output minus its start in the tile
  __shared__ unsigned buf[RS_TILE];          // exchange buffer
  __shared__ unsigned wsum[RADIX / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < RS_WARPS * RADIX; i += RS_THREADS) (&cnt[0][0])[i] = 0;
  __syncthreads();
  const i64 tbase = (i64)blockIdx.x * RS_TILE;
  const i64 wbase = tbase + (i64)warp * RS_WARP_ITEMS;
  const int n_tile = (int)(n - tbase < RS_TILE ? n - tbase : RS_TILE);
  unsigned key[RS_IPT];
  unsigned lpos[RS_IPT];  // rank among the warp's items of the same digit, then position in the sorted tile
#pragma unroll
  for (int t = 0; t < RS_IPT; ++t) {
    const i64 idx = wbase + t * 32 + lane;
    key[t] = idx < n ? __ldg(keys_in + idx) : 0u;
  }
#pragma unroll
  for (int t = 0; t < RS_IPT; ++t) {
    const bool valid = wbase + t * 32 + lane < n;
    const unsigned d = (key[t] >> shift) & (RADIX - 1);
    const unsigned peers = __match_any_sync(DGNN_FULL, valid ? d : (unsigned)RADIX);
    const int leader = __ffs(peers) - 1;
    unsigned base = 0;
    if (lane == leader && valid) {
      base = cnt[warp][d];
      cnt[warp][d] = base + __popc(peers);
    }
    base = __shfl_sync(DGNN_FULL, base, leader);
    lpos[t] = base + __popc(peers & ((1u << lane) - 1u));
    __syncwarp();
  }
  __syncthreads();
  unsigned total = 0, incl = 0;
  if (tid < RADIX) {  // exclusive prefix of digit tid over the warps, and the digit's total
#pragma unroll
    for (int w = 0; w < RS_WARPS; ++w) {
      const unsigned c = cnt[w][tid];
      cnt[w][tid] = total;
      total += c;
    }
    incl = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned v = __shfl_up_sync(DGNN_FULL, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
  }
  __syncthreads();
  if (tid < RADIX) {
    unsigned lstart = incl - total;  // where the digit's run starts in the sorted tile
    for (int w = 0; w < warp; ++w) lstart += wsum[w];
    gbase[tid] = tile_off[(i64)tid * ntiles + blockIdx.x] - lstart;
#pragma unroll
    for (int w = 0; w < RS_WARPS; ++w) cnt[w][tid] += lstart;
  }
  __syncthreads();
#pragma unroll
  for (int t = 0; t < RS_IPT; ++t) {
    if (wbase + t * 32 + lane < n) {
      lpos[t] += cnt[warp][(key[t] >> shift) & (RADIX - 1)];
      buf[lpos[t]] = key[t];
    }
  }
  __syncthreads();
  unsigned dst[RS_IPT];
#pragma unroll
  for (int k = 0; k < RS_IPT; ++k) {
    const int i = k * RS_THREADS + tid;
    if (i < n_tile) {
      const unsigned kk = buf[i];
      dst[k] = gbase[(kk >> shift) & (RADIX - 1)] + (unsigned)i;
      keys_out[dst[k]] = kk;
    }
  }
  __syncthreads();
  // payload 1: CSR position
#pragma unroll
  for (int t = 0; t < RS_IPT; ++t) {
    const i64 idx = wbase + t * 32 + lane;
    if (idx < n) buf[lpos[t]] = FIRST ? (unsigned)idx : (unsigned)__ldg(pos_in + idx);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < RS_IPT; ++k) {
    const int i = k * RS_THREADS + tid;
    if (i < n_tile) pos_out[dst[k]] = (int)buf[i];
  }
  if (!TWO) return;
  __syncthreads();
  // payload 2: row id (FIRST: looked up between the rows of the warp's first and last entry)
  i64 r_lo = 0, r_hi = 0;
  if (FIRST && wbase < n) {
    const i64 gw = wbase / RS_WARP_ITEMS;
    r_lo = __ldg(wrow + gw);
    r_hi = wbase + RS_WARP_ITEMS < n ? (i64)__ldg(wrow + gw + 1) : n_rows - 1;   // row of the next run's first entry bounds this run's rows
  }
#pragma unroll
  for (int t = 0; t < RS_IPT; ++t) {
    const i64 idx = wbase + t * 32 + lane;
    if (idx >= n) continue;
    int row;
    if (FIRST) {
      i64 lo = r_lo, hi = r_hi + 1;  // row_ptr[lo] <= idx < row_ptr[hi]
      while (hi - lo > 1) {
        const i64 mid = (lo + hi) >> 1;
        if (ldp(row_ptr, idx_bits, mid) <= idx) lo = mid; else hi = mid;
      }
      row = (int)lo;
    } else {
      row = __ldg(row_in + idx);
    }
    buf[lpos[t]] = (unsigned)row;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < RS_IPT; ++k) {
    const int i = k * RS_THREADS + tid;
    if (i < n_tile) row_out[dst[k]] = (int)buf[i];
  }
}

__global__ void k_coo2csr(i64 nnz, i64 m, const int* row_ind, void* row_ptr, int bits) {
  const i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (i > m) return;
  i64 lo = 0, hi = nnz;  // first position whose row id is >= i
  while (lo < hi) {
    const i64 mid = (lo + hi) >> 1;
    if ((i64)__ldg(row_ind + mid) < i) lo = mid + 1; else hi = mid;
  }
  if (bits == 64) reinterpret_cast<i64*>(row_ptr)[i] = lo;
  else reinterpret_cast<int*>(row_ptr)[i] = (int)lo;
}

struct C2CLayout {
  size_t tile_hist, scan_scratch, wrow, keys[2], pos[2], row[2], total;
  i64 ntiles;
  int passes;
};
inline C2CLayout c2c_layout(i64 n_cols, i64 nnz) {
  C2CLayout L;
  int bits = 1;
  while (((i64)1 << bits) < n_cols) ++bits;
  L.passes = (bits + 7) / 8;
  L.ntiles = cdiv(nnz > 0 ? nnz : 1, RS_TILE);
  const i64 hist_items = (i64)RADIX * L.ntiles;
  size_t off = 0;
  L.tile_hist = off;    off += up256((size_t)hist_items * 4);
  L.scan_scratch = off; off += up256((size_t)scan_scratch_items(hist_items) * 4);
  L.wrow = off;         off += up256((size_t)(cdiv(nnz > 0 ? nnz : 1, RS_WARP_ITEMS) + 1) * 4);
  for (int i = 0; i < 2; ++i) {
    // pass p writes slot p & 1: the keys of every pass (the last pass's sorted ids give col_ptr), the
    // payload of every pass but the last (that one goes to permute / row_ind)
    const bool need_keys = L.passes > i, need_payload = L.passes > i + 1;
    L.keys[i] = off; off += need_keys ? up256((size_t)nnz * 4) : 0;
    L.pos[i] = off;  off += need_payload ? up256((size_t)nnz * 4) : 0;
    L.row[i] = off;  off += need_payload ? up256((size_t)nnz * 4) : 0;
  }
  L.total = off + 256;
  return L;
}

}  // namespace

// implementation shared with the allocation-free entry point
int dgnn_csr2csc_impl(i64 n_rows, i64 n_cols, i64 nnz, const void* row_ptr, int idx_bits,
                      const int32_t* col_ind, void* col_ptr, int32_t* row_ind, int32_t* permute,
                      char* wsb, cudaStream_t s) {
  const C2CLayout L = c2c_layout(n_cols, nnz);
  unsigned* tile_hist = reinterpret_cast<unsigned*>(wsb + L.tile_hist);
  unsigned* scratch = reinterpret_cast<unsigned*>(wsb + L.scan_scratch);
  int* wrow = reinterpret_cast<int*>(wsb + L.wrow);
  const unsigned* sorted = nullptr;
  if (nnz > 0) {
    k_warp_rows<<<dgnn_grid(cdiv(nnz, RS_WARP_ITEMS), 256), 256, 0, s>>>(nnz, n_rows, row_ptr, idx_bits, wrow, RS_WARP_ITEMS);
    const unsigned* kin = reinterpret_cast<const unsigned*>(col_ind);
    const int* pin = nullptr;
    const int* rin = nullptr;
    const unsigned grid = (unsigned)L.ntiles;
    for (int p = 0; p < L.passes; ++p) {
      const bool first = p == 0, last = p == L.passes - 1;
      const int shift = 8 * p;
      unsigned* kout = reinterpret_cast<unsigned*>(wsb + L.keys[p & 1]);
      int* pout = last ? permute : reinterpret_cast<int*>(wsb + L.pos[p & 1]);
      int* rout = last ? row_ind : reinterpret_cast<int*>(wsb + L.row[p & 1]);
      k_radix_hist<<<grid, HIST_THREADS, 0, s>>>(kin, nnz, shift, tile_hist, L.ntiles);
      int rc = exclusive_scan(tile_hist, (i64)RADIX * L.ntiles, scratch, s);
      if (rc) return rc;
#define RS_ARGS kin, pin, rin, kout, pout, rout, nnz, shift, tile_hist, L.ntiles, row_ptr, idx_bits, n_rows, wrow
      if (first) k_radix_scatter<true, true><<<grid, RS_THREADS, 0, s>>>(RS_ARGS);
      else k_radix_scatter<false, true><<<grid, RS_THREADS, 0, s>>>(RS_ARGS);
#undef RS_ARGS
      kin = kout; pin = pout; rin = rout;
    }
    sorted = kin;
  }
  k_col_ptr<<<dgnn_grid(n_cols + 1, 256), 256, 0, s>>>(n_cols, nnz, sorted, col_ptr, idx_bits);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

size_t dgnn_csr2csc_scratch_bytes(i64 n_cols, i64 nnz) { return c2c_layout(n_cols, nnz).total; }

// ---------------------------------------------------------------------------
// Stable sort of (key, value) pairs by the low key_bits bits of the key with the same radix passes; two of
// them in a row (by source, then by destination) order an edge list by (destination, source).
// ---------------------------------------------------------------------------
namespace {
struct PairLayout {
  size_t tile_hist, scan_scratch, keys, vals, total;
  i64 ntiles;
  int passes;
};
inline PairLayout pair_layout(i64 n, int key_bits) {
  PairLayout L;
  L.passes = (key_bits + 7) / 8;
  if (L.passes < 1) L.passes = 1;
  L.ntiles = cdiv(n > 0 ? n : 1, RS_TILE);
  const i64 hist_items = (i64)RADIX * L.ntiles;
  size_t off = 0;
  L.tile_hist = off;    off += up256((size_t)hist_items * 4);
  L.scan_scratch = off; off += up256((size_t)scan_scratch_items(hist_items) * 4);
  L.keys = off;         off += up256((size_t)n * 4);      // one ping-pong partner: the output arrays are the other
  L.vals = off;         off += up256((size_t)n * 4);
  L.total = off + 256;
  return L;
}

// passes alternate between (tmp) and (out); the last one lands in out
int sort_pairs(i64 n, int key_bits, const unsigned* keys_in, const int* vals_in, unsigned* keys_out, int* vals_out,
               char* wsb, cudaStream_t s) {
  const PairLayout L = pair_layout(n, key_bits);
  unsigned* tile_hist = reinterpret_cast<unsigned*>(wsb + L.tile_hist);
  unsigned* scratch = reinterpret_cast<unsigned*>(wsb + L.scan_scratch);
  unsigned* ktmp = reinterpret_cast<unsigned*>(wsb + L.keys);
  int* vtmp = reinterpret_cast<int*>(wsb + L.vals);
  const unsigned* kin = keys_in;
  const int* vin = vals_in;
  const unsigned grid = (unsigned)L.ntiles;
  for (int p = 0; p < L.passes; ++p) {
    const bool to_out = ((L.passes - 1 - p) & 1) == 0;
    unsigned* kout = to_out ? keys_out : ktmp;
    int* vout = to_out ? vals_out : vtmp;
    k_radix_hist<<<grid, HIST_THREADS, 0, s>>>(kin, n, 8 * p, tile_hist, L.ntiles);
    int rc = exclusive_scan(tile_hist, (i64)RADIX * L.ntiles, scratch, s);
    if (rc) return rc;
    k_radix_scatter<false, false><<<grid, RS_THREADS, 0, s>>>(kin, vin, nullptr, kout, vout, nullptr, n, 8 * p, tile_hist,
                                                               L.ntiles, nullptr, 32, 0, nullptr);
    kin = kout; vin = vout;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}
}  // namespace

// ---------------------------------------------------------------------------
// Allocation-free variant: the scratch of the conversion lives in a fixed array
// inside the library image instead of a caller-supplied workspace.
// ---------------------------------------------------------------------------
constexpr i64 STATIC_MAX_NNZ = 1 << 20;    // entries
constexpr i64 STATIC_MAX_COLS = 1 << 20;   // columns
constexpr size_t STATIC_SCRATCH_BYTES = size_t(32) << 20;  // 32 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_csr2csc_scratch[STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_static_mu;
char* g_static_ptr[MAX_DEVICES] = {nullptr};

// The symbol name is only a host-side handle; the device address has to be asked
// for, once per device, while that device is current.
int static_scratch_for_current_device(char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return DGNN_ERR_VALUE;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_csr2csc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_ptr[dev] = static_cast<char*>(p);
  }
  *out = g_static_ptr[dev];
  return DGNN_OK;
}
}  // namespace

extern "C" {

size_t dgnn_csr2csc_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz) {
  (void)n_rows;
  if (n_cols < 0 || nnz < 0) return 256;
  return c2c_layout(n_cols, nnz).total;
}

int dgnn_csr2csc(int64_t n_rows, int64_t n_cols, int64_t nnz, const void* row_ptr, int idx_bits,
                 const int32_t* col_ind, void* col_ptr, int32_t* row_ind, int32_t* permute,
                 void* workspace, size_t workspace_bytes, void* stream) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return DGNN_ERR_SHAPE;
  if (idx_bits != 32 && idx_bits != 64) return DGNN_ERR_IDX_BITS;
  if (nnz > 0x7fffffffLL || n_rows > 0x7fffffffLL || n_cols > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (!row_ptr || !col_ptr || (nnz > 0 && (!col_ind || !row_ind || !permute))) return DGNN_ERR_NULL;
  if (!workspace || workspace_bytes < c2c_layout(n_cols, nnz).total) return DGNN_ERR_WORKSPACE;
  char* wsb = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  return dgnn_csr2csc_impl(n_rows, n_cols, nnz, row_ptr, idx_bits, col_ind, col_ptr, row_ind, permute, wsb,
                           reinterpret_cast<cudaStream_t>(stream));
}

size_t dgnn_coo_sort_workspace_bytes(int64_t nnz, int64_t n_nodes) {
  if (nnz < 0 || n_nodes < 0) return 256;
  int bits = 1;
  while (((i64)1 << bits) < n_nodes) ++bits;
  return pair_layout(nnz, bits).total + 2 * up256((size_t)nnz * 4);
}

int dgnn_coo_sort(int64_t nnz, int64_t n_nodes, const int32_t* dst, const int32_t* src, int32_t* dst_sorted,
                  int32_t* src_sorted, void* workspace, size_t workspace_bytes, void* stream) {
  if (nnz < 0 || n_nodes < 0) return DGNN_ERR_SHAPE;
  if (nnz > 0x7fffffffLL || n_nodes > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (nnz == 0) return DGNN_OK;
  if (!dst || !src || !dst_sorted || !src_sorted) return DGNN_ERR_NULL;
  if (!workspace || workspace_bytes < dgnn_coo_sort_workspace_bytes(nnz, n_nodes)) return DGNN_ERR_WORKSPACE;
  int bits = 1;
  while (((i64)1 << bits) < n_nodes) ++bits;
  char* wsb = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  const PairLayout L = pair_layout(nnz, bits);
  unsigned* mid_src = reinterpret_cast<unsigned*>(wsb + L.total);
  int* mid_dst = reinterpret_cast<int*>(wsb + L.total + up256((size_t)nnz * 4));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // by source (destination rides along), then stably by destination (source rides along)
  int rc = sort_pairs(nnz, bits, reinterpret_cast<const unsigned*>(src), dst, mid_src, mid_dst, wsb, s);
  if (rc) return rc;
  return sort_pairs(nnz, bits, reinterpret_cast<const unsigned*>(mid_dst), reinterpret_cast<const int*>(mid_src),
                    reinterpret_cast<unsigned*>(dst_sorted), src_sorted, wsb, s);
}

int dgnn_coo2csr(int64_t nnz, int64_t m, const int32_t* row_ind, void* row_ptr, int idx_bits, void* stream) {
  if (nnz < 0 || m < 0) return DGNN_ERR_SHAPE;
  if (idx_bits != 32 && idx_bits != 64) return DGNN_ERR_IDX_BITS;
  if (idx_bits == 32 && nnz > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (!row_ptr || (nnz > 0 && !row_ind)) return DGNN_ERR_NULL;
  k_coo2csr<<<dgnn_grid(m + 1, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(nnz, m, row_ind, row_ptr, idx_bits);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

int64_t dgnn_csr2csc_static_max_nnz(void) { return STATIC_MAX_NNZ; }
int64_t dgnn_csr2csc_static_max_cols(void) { return STATIC_MAX_COLS; }

int dgnn_csr2csc_static(int64_t n_rows, int64_t n_cols, int64_t nnz, const void* row_ptr, int idx_bits,
                        const int32_t* col_ind, void* col_ptr, int32_t* row_ind, int32_t* permute, void* stream) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return DGNN_ERR_SHAPE;
  if (idx_bits != 32 && idx_bits != 64) return DGNN_ERR_IDX_BITS;
  if (n_rows > 0x7fffffffLL) return DGNN_ERR_OVERFLOW;
  if (nnz > STATIC_MAX_NNZ || n_cols > STATIC_MAX_COLS) return DGNN_ERR_STATIC_LIMIT;
  if (c2c_layout(n_cols, nnz).total > STATIC_SCRATCH_BYTES) return DGNN_ERR_STATIC_LIMIT;
  if (!row_ptr || !col_ptr || (nnz > 0 && (!col_ind || !row_ind || !permute))) return DGNN_ERR_NULL;
  char* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  // every region of the scratch that is read is written first by this call (tile histograms, row
  // table and the ping-pong buffers are all overwritten before use), so stale contents of the previous
  // call do no harm and nothing needs clearing
  return dgnn_csr2csc_impl(n_rows, n_cols, nnz, row_ptr, idx_bits, col_ind, col_ptr, row_ind, permute, scratch,
                           reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"

// Shared device helpers for the dgnn_b200 kernels (sm_100a).
//
// Scheduling model used by every per-row (or per-column) operator in this
// library: rows whose degree is at most SEG edges are handled by one warp each
// (k_rows).  Longer rows are cut at the global edge positions that are
// multiples of SEG; every (chunk, row) piece is handled by one warp (k_chunks)
// that writes a partial state to a workspace slot, and one warp per long row
// (k_merge) folds the partials in edge order.  A chunk of SEG edges can meet at
// most two long rows -- one that began before the chunk (slot 0) and one that
// begins inside it (slot 1) -- so the workspace needs 2 * ceil(nnz / SEG)
// slots and no atomics, and the result does not depend on scheduling.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/dgnn_b200.h"

typedef long long i64;

#define DGNN_FULL 0xffffffffu
constexpr int DGNN_SEG = 1024;         // edges per chunk for long-row splitting
constexpr int DGNN_WARPS = 8;          // warps per CTA in the row kernels
constexpr int DGNN_THREADS = DGNN_WARPS * 32;
constexpr int DGNN_ROW_WARPS = 4;      // warps per CTA in the strided short-row kernel
constexpr int DGNN_ROW_THREADS = DGNN_ROW_WARPS * 32;
constexpr i64 DGNN_SMALL_NNZ = 16 * 1024;  // graphs up to this many entries run as one launch per operator
constexpr int DGNN_CHUNK_WARPS = 4;    // warps that share one (chunk, long row) piece
constexpr float DGNN_NEG_INIT = -1e38f;  // initial running maximum (matches the reference)

// index-pointer arrays come as int32 or int64; the width is uniform per launch
__device__ __forceinline__ i64 ldp(const void* p, int bits, i64 i) {
  return bits == 64 ? __ldg(reinterpret_cast<const i64*>(p) + i)
                    : (i64)__ldg(reinterpret_cast<const int*>(p) + i);
}

// row r with indptr[r] <= pos < indptr[r+1]; requires 0 <= pos < indptr[n_rows]
__device__ __forceinline__ i64 find_row(const void* indptr, int bits, i64 n_rows, i64 pos) {
  i64 lo = 0, hi = n_rows;
  while (hi - lo > 1) {
    i64 mid = (lo + hi) >> 1;
    if (ldp(indptr, bits, mid) <= pos) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ float4 ld4(const float4* p) { return __ldg(p); }
// load of a gathered row (one per edge).  Through the L1 like any read-only load: the hub rows of a skewed graph are
// re-read by the same SM often enough that caching at the L2 only (ld.global.cg: +2 % on the forward and backward
// sweeps at R-MAT 2.4 M / 120 M) or L1::no_allocate (+11-14 %) is slower.
__device__ __forceinline__ float4 ld4_gather(const float4* p) { return __ldg(p); }
// 32 contiguous bytes per lane in one instruction (the 256-bit global loads and stores of sm_100); p must be
// 32-byte aligned.  A warp then fetches a 1 KB row with one request instead of two: on the GAT sweeps, whose first
// limit is the L1TEX data pipe, that is 5-6 % of the forward and the backward sweep.
__device__ __forceinline__ void ld8_gather(const float4* p, float4& a, float4& b) {
  asm("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w), "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w) : "l"(p));
}
__device__ __forceinline__ void st8(float4* p, const float4& a, const float4& b) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               :: "l"(p), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w), "f"(b.x), "f"(b.y), "f"(b.z), "f"(b.w) : "memory");
}
// Read-only load whose line is the last to leave the L2: for the rows of a gathered tensor that many edges
// reference (the "hot" rows, see dgnn_hot_rows).  A feature tensor of gigabytes streams through the 126 MB L2;
// with plain loads the often-referenced rows are evicted by rows that are read once.
__device__ __forceinline__ unsigned long long l2_keep_policy() {
  unsigned long long pol;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ float4 ld4_keep(const float4* p, unsigned long long pol) {
  float4 v;
  asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
      : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(pol));
  return v;
}
__device__ __forceinline__ void ld8_keep(const float4* p, float4& a, float4& b, unsigned long long pol) {
  asm("ld.global.nc.L2::cache_hint.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8], %9;"
      : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w), "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w) : "l"(p), "l"(pol));
}
__device__ __forceinline__ float ld1_keep(const float* p, unsigned long long pol) {
  float v;
  asm("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
  return v;
}
#ifndef DGNN_STREAM_STORES
#define DGNN_STREAM_STORES 1
#endif
#ifndef DGNN_STREAM_INDEX
#define DGNN_STREAM_INDEX 1
#endif
// store of a result that this kernel does not read again: first in line to leave the L2
__device__ __forceinline__ void st4_stream(float4* p, const float4& v) {
#if DGNN_STREAM_STORES
  __stcs(p, v);
#else
  *p = v;
#endif
}
// an index array entry that is read once
__device__ __forceinline__ int ld_index(const int* p) {
#if DGNN_STREAM_INDEX
  return __ldcs(p);
#else
  return __ldg(p);
#endif
}
// the hot flag of a gathered row travels in the sign bit of its (non-negative int32) index
__device__ __forceinline__ int dgnn_tag_hot(const unsigned* hot, int idx) {
  return hot ? (idx | (int)(((__ldg(hot + (idx >> 5)) >> (idx & 31)) & 1u) << 31)) : idx;
}
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }
// Packed fp32 arithmetic (fma.rn.f32x2 / mul.rn.f32x2 of sm_100: two lanes per issued instruction, each rounded as
// the scalar operation, so the results are bit-identical).  Off: measured on the GAT sweeps it changes nothing (their
// first limit is the L1TEX data pipe, not the issue rate), and the register pairs it needs cost the streaming
// kernels occupancy (logits backward 62 -> 74 registers, 1.19 -> 1.64 ms at 2.4 M rows x 8 heads x 32).
#ifndef DGNN_FFMA2
#define DGNN_FFMA2 0
#endif
__device__ __forceinline__ void fma4(float4& acc, float w, const float4& x) {
#if DGNN_FFMA2
  const float2 ww = make_float2(w, w);
  const float2 lo = __ffma2_rn(ww, make_float2(x.x, x.y), make_float2(acc.x, acc.y));
  const float2 hi = __ffma2_rn(ww, make_float2(x.z, x.w), make_float2(acc.z, acc.w));
  acc = make_float4(lo.x, lo.y, hi.x, hi.y);
#else
  acc.x = fmaf(w, x.x, acc.x); acc.y = fmaf(w, x.y, acc.y);
  acc.z = fmaf(w, x.z, acc.z); acc.w = fmaf(w, x.w, acc.w);
#endif
}
__device__ __forceinline__ void scale4(float4& a, float s) {
#if DGNN_FFMA2
  const float2 ss = make_float2(s, s);
  const float2 lo = __fmul2_rn(ss, make_float2(a.x, a.y)), hi = __fmul2_rn(ss, make_float2(a.z, a.w));
  a = make_float4(lo.x, lo.y, hi.x, hi.y);
#else
  a.x *= s; a.y *= s; a.z *= s; a.w *= s;
#endif
}
__device__ __forceinline__ void add4(float4& a, const float4& b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
  return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}
// t += (a.x*b.x + a.z*b.z, a.y*b.y + a.w*b.w): a dot product kept as two partial sums (t.x + t.y at the end)
__device__ __forceinline__ void dot4_acc(float2& t, const float4& a, const float4& b) {
#if DGNN_FFMA2
  t = __ffma2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y), t);
  t = __ffma2_rn(make_float2(a.z, a.w), make_float2(b.z, b.w), t);
#else
  t.x = fmaf(a.z, b.z, fmaf(a.x, b.x, t.x));
  t.y = fmaf(a.w, b.w, fmaf(a.y, b.y, t.y));
#endif
}
__device__ __forceinline__ float leaky(float x, float slope) { return x > 0.f ? x : x * slope; }
// exp through the hardware ex2 unit: relative error ~2^-22 plus |x| * 2^-24 from the
// log2(e) scaling, far inside the fp32 tolerance of the operators (1e-4 relative)
__device__ __forceinline__ float fast_exp(float x) { return __expf(x); }

// Feature rows are H*F floats viewed as HF4 = H*F/4 float4 vectors.  With LPR = 32
// lane l owns vectors q = l + 32*v (v < VPL); vector q belongs to head q >> f4_shift
// where 2^f4_shift = F/4 vectors per head.  Narrow rows (HF4 <= 16, VPL = 1) use
// LPR = 16 or 8 lanes per row: the warp is cut into 32/LPR sub-groups that work on
// different edges of the same row at the same time (sub-group sg takes every
// (32/LPR)-th edge) and fold their states at the end of the row, so no lane idles.
template <int VPL, int LPR = 32>
struct LaneMap {
  static_assert(LPR == 32 || VPL == 1, "sub-groups only for rows of at most 32 vectors");
  static constexpr int EPW = 32 / LPR;  // edges a warp works on per step
  int sg;          // sub-group of this lane
  int q[VPL];
  int hd[VPL];
  bool act[VPL];
  bool lead[VPL];   // first vector of its head (in its sub-group)
  bool wr[VPL];     // this lane writes the row's vector q (sub-group 0 only)
  bool wlead[VPL];  // this lane writes the per-head scalars of the row
  __device__ __forceinline__ void init(int lane, int hf4, int f4_shift) {
    sg = lane / LPR;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      q[v] = (lane % LPR) + LPR * v;
      act[v] = q[v] < hf4;
      hd[v] = act[v] ? (q[v] >> f4_shift) : 0;
      lead[v] = act[v] && ((q[v] & ((1 << f4_shift) - 1)) == 0);
      wr[v] = act[v] && sg == 0;
      wlead[v] = lead[v] && sg == 0;
    }
  }
};

// Sum p[u][v] over all vectors of the same head, for U independent edges at once;
// every lane of the head ends with the total.  All 32 lanes must call it.  The
// butterfly steps are compile-time offsets under a uniform predicate, and each step
// is issued for all U*VPL values before the next one so the shuffles overlap.
template <int U, int VPL>
__device__ __forceinline__ void head_reduce(float (&p)[U][VPL], int f4_shift) {
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    if (s < f4_shift) {
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int v = 0; v < VPL; ++v) p[u][v] += __shfl_xor_sync(DGNN_FULL, p[u][v], 1 << s);
    }
  }
  if (f4_shift > 5) {
    const int g = 1 << (f4_shift - 5);  // vector slots per head
#pragma unroll
    for (int s = 1; s < VPL; s <<= 1) {
      if (s < g) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float t[VPL];
#pragma unroll
          for (int v = 0; v < VPL; ++v) t[v] = p[u][v] + p[u][v ^ s];
#pragma unroll
          for (int v = 0; v < VPL; ++v) p[u][v] = t[v];
        }
      }
    }
  }
}
template <int VPL>
__device__ __forceinline__ void head_reduce(float (&p)[VPL], int f4_shift) {
  float q[1][VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) q[0][v] = p[v];
  head_reduce<1, VPL>(q, f4_shift);
#pragma unroll
  for (int v = 0; v < VPL; ++v) p[v] = q[0][v];
}

// ---------------------------------------------------------------------------
// the three scheduling kernels, generic over an operator object
// Op must provide: n_rows, nnz, indptr, idx_bits, ws (float* partial slots),
//   slot_stride (floats per slot), MIN_BLOCKS, HAS_PARTIALS, struct State,
//   skip_empty (rows without edges need no work), init(State&, row, lane) = empty state,
//   STAGED (bool; true: members first, last, stage, stage_mask -- see dgnn_row_role),
//   resume(State&, row, lane, first) = unless first, fold in a state carried from an earlier call (once per row),
//   ring_bytes() = shared memory per warp for an operator that stages its gathered rows there (0: none),
//   range(State&, row, e0, e1, lane, ring) with ring = the warp's staging area,
//   combine(State&, lane) = fold the sub-groups' states after range,
//   finalize(State&, row, lane, last) = write the row's result (last) or its state, store_partial(State&, float* p, lane),
//   merge_partial(State&, const float* p, lane)
// ---------------------------------------------------------------------------
// The part a row plays in this launch.  Plain operators: the whole row, once (first = last = true).  Staged
// sweeps (Op::STAGED) carry a per-row state between launches: either every row takes part in every stage
// (op.first / op.last mark the ends), or -- with op.stage_mask -- bit p of stage_mask[r] says whether row r has
// entries in stage p: the row starts fresh in its first such stage, is written out in its last one and is not
// touched (no state read or written) in any other; rows without entries anywhere are written by stage 0.
template <class Op>
__device__ __forceinline__ bool dgnn_row_role(const Op& op, i64 r, bool& first, bool& last) {
  if constexpr (Op::STAGED) {
    if (op.stage_mask == nullptr) {
      first = op.first != 0;
      last = op.last != 0;
      return true;
    }
    const unsigned m = op.stage_mask[r];
    const int p = op.stage;
    if (m == 0) {
      first = last = true;
      return p == 0;
    }
    first = (m & ((1u << p) - 1u)) == 0;
    last = (m >> (p + 1)) == 0;
    return ((m >> p) & 1u) != 0;
  } else {
    first = last = true;
    return true;
  }
}

// Short rows: every warp of a fixed pool draws the next `batch` rows (1..31) from a
// counter.  Rows come out in id order, so whatever skew the ids carry (R-MAT: low
// ids are the heavy ones) is spread over all warps and the tail consists of a few
// rows.  The batch grows as the average row gets shorter, which keeps the rate of
// atomics on the one counter far below what the memory system serialises, and the
// batch's index pointers arrive in one coalesced load.
// Rows of more than DGNN_HEAVY entries are handled first (pass 0), all others afterwards (pass 1); a warp goes on to
// pass 1 as soon as pass 0 has no draws left, there is no barrier in between.  A row is one warp's work from its
// first entry to its last (about 0.4 us per entry in the GAT sweeps), so the last rows to be drawn decide how long
// the grid idles at its end: with the heavy rows out of the way that is a row of at most DGNN_HEAVY entries instead
// of one of up to DGNN_SEG.  A draw of pass 0 looks at 31 rows spread evenly over the whole id range (row b, b + nb,
// b + 2 nb, ...: where heavy rows cluster at some ids, as the low ids of an R-MAT graph, consecutive rows would give
// one warp dozens of them) and handles the heavy ones; pass 1 draws `batch` consecutive rows and skips the heavy ones.
#ifndef DGNN_HEAVY_ROWS
#define DGNN_HEAVY_ROWS 128
#endif
constexpr int DGNN_HEAVY = DGNN_HEAVY_ROWS;

template <class Op>
__device__ __forceinline__ void dgnn_one_row(const Op& op, i64 r, i64 lb, i64 hb, int lane, float4* ring) {
  bool first, last;
  if (!dgnn_row_role(op, r, first, last)) return;
  typename Op::State st;
  op.init(st, r, lane);
  op.resume(st, r, lane, first);
  op.range(st, r, lb, hb, lane, ring);
  op.combine(st, lane);
  op.finalize(st, r, lane, last);
}

template <class Op>
__global__ void __launch_bounds__(DGNN_ROW_THREADS, Op::MIN_BLOCKS) k_rows(const Op op, unsigned long long* next_row, const int batch) {
  extern __shared__ float4 dgnn_smem4[];
  const int lane = threadIdx.x & 31;
  float4* ring = dgnn_smem4 + (size_t)(threadIdx.x >> 5) * (op.ring_bytes() / 16);
  // pass 0: heavy rows, 31 strided rows per draw
  const i64 nb = (op.n_rows + 30) / 31;
  for (;;) {
    unsigned long long t = 0;
    if (lane == 0) t = atomicAdd(next_row, 1ull);
    const i64 b = (i64)__shfl_sync(DGNN_FULL, t, 0);
    if (b >= nb) break;
    const i64 mine_r = b + (i64)lane * nb;
    const bool valid = lane < 31 && mine_r < op.n_rows;
    const i64 lo = valid ? ldp(op.indptr, op.idx_bits, mine_r) : 0;
    const i64 hi = valid ? ldp(op.indptr, op.idx_bits, mine_r + 1) : 0;
    unsigned todo = __ballot_sync(DGNN_FULL, valid && hi - lo > DGNN_HEAVY && hi - lo <= DGNN_SEG);
    while (todo) {
      const int i = __ffs(todo) - 1;
      todo &= todo - 1;
      dgnn_one_row(op, b + (i64)i * nb, __shfl_sync(DGNN_FULL, lo, i), __shfl_sync(DGNN_FULL, hi, i), lane, ring);
    }
  }
  // pass 1: everything else, `batch` consecutive rows per draw
  for (;;) {
    unsigned long long t = 0;
    if (lane == 0) t = atomicAdd(next_row + 1, (unsigned long long)batch);
    const i64 r0 = (i64)__shfl_sync(DGNN_FULL, t, 0);
    if (r0 >= op.n_rows) break;
    const int cnt = (int)((op.n_rows - r0 < batch) ? op.n_rows - r0 : batch);
    const i64 mine = lane <= cnt ? ldp(op.indptr, op.idx_bits, r0 + lane) : 0;
    const i64 len = __shfl_down_sync(DGNN_FULL, mine, 1) - mine;   // lane i < cnt: length of row r0 + i
    // long rows belong to the chunk + merge kernels; empty rows of a middle stage keep their carried state
    unsigned todo = __ballot_sync(DGNN_FULL, lane < cnt && len <= DGNN_HEAVY && !(op.skip_empty && len == 0));
    while (todo) {
      const int i = __ffs(todo) - 1;
      todo &= todo - 1;
      dgnn_one_row(op, r0 + i, __shfl_sync(DGNN_FULL, mine, i), __shfl_sync(DGNN_FULL, mine, i + 1), lane, ring);
    }
  }
}

// Small graphs (at most DGNN_SMALL_NNZ entries): one launch, one warp per row whatever its
// length, no counter and no chunk / merge kernels -- launch latency is all that matters there.
template <class Op>
__global__ void __launch_bounds__(DGNN_ROW_THREADS, Op::MIN_BLOCKS) k_rows_small(const Op op) {
  extern __shared__ float4 dgnn_smem4[];
  const int lane = threadIdx.x & 31;
  float4* ring = dgnn_smem4 + (size_t)(threadIdx.x >> 5) * (op.ring_bytes() / 16);
  const i64 r = (i64)blockIdx.x * DGNN_ROW_WARPS + (threadIdx.x >> 5);
  if (r >= op.n_rows) return;
  const i64 lb = ldp(op.indptr, op.idx_bits, r);
  const i64 hb = ldp(op.indptr, op.idx_bits, r + 1);
  if (op.skip_empty && hb == lb) return;
  bool first, last;
  if (!dgnn_row_role(op, r, first, last)) return;
  typename Op::State st;
  op.init(st, r, lane);
  op.resume(st, r, lane, first);
  op.range(st, r, lb, hb, lane, ring);
  op.combine(st, lane);
  op.finalize(st, r, lane, last);
}

// Long rows: one CTA of DGNN_CHUNK_WARPS warps per (chunk, slot).  The piece of the
// row inside the chunk is cut into equal sub-ranges, one per warp; the warps'
// states are folded in edge order through shared memory and warp 0 writes the
// chunk's partial state.
template <class Op>
__global__ void __launch_bounds__(DGNN_CHUNK_WARPS * 32, Op::MIN_BLOCKS) k_chunks(const Op op) {
  extern __shared__ float4 dgnn_smem4[];   // [partial states of warps 1.. | staging areas of the warps]
  float* smem = reinterpret_cast<float*>(dgnn_smem4);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t part4 = Op::HAS_PARTIALS ? ((size_t)(DGNN_CHUNK_WARPS - 1) * op.slot_stride + 3) / 4 : 0;
  float4* ring = dgnn_smem4 + part4 + (size_t)warp * (op.ring_bytes() / 16);
  const i64 w = blockIdx.x;
  const i64 j = w >> 1;
  const int slot = (int)(w & 1);
  const i64 cs = j * DGNN_SEG;
  if (cs >= op.nnz) return;
  const i64 ce = (cs + DGNN_SEG < op.nnz) ? cs + DGNN_SEG : op.nnz;
  const i64 r = find_row(op.indptr, op.idx_bits, op.n_rows, slot ? ce - 1 : cs);
  const i64 lb = ldp(op.indptr, op.idx_bits, r);
  const i64 hb = ldp(op.indptr, op.idx_bits, r + 1);
  if (hb - lb <= DGNN_SEG) return;
  if (slot == 0 ? (lb >= cs) : (lb < cs)) return;
  const i64 e0 = lb > cs ? lb : cs, e1 = hb < ce ? hb : ce;
  const i64 per = (e1 - e0 + DGNN_CHUNK_WARPS - 1) / DGNN_CHUNK_WARPS;
  const i64 w0 = e0 + per * warp;
  const i64 w1 = (w0 + per < e1) ? w0 + per : e1;
  typename Op::State st;
  op.init(st, r, lane);
  if (w0 < w1) op.range(st, r, w0, w1, lane, ring);
  if (!Op::HAS_PARTIALS) return;
  op.combine(st, lane);
  if (warp > 0) op.store_partial(st, smem + (i64)(warp - 1) * op.slot_stride, lane);
  __syncthreads();
  if (warp == 0) {
    for (int k = 1; k < DGNN_CHUNK_WARPS; ++k)
      if (e0 + per * k < e1) op.merge_partial(st, smem + (i64)(k - 1) * op.slot_stride, lane);
    op.store_partial(st, op.ws + (2 * j + slot) * op.slot_stride, lane);
  }
}

template <class Op>
__global__ void __launch_bounds__(DGNN_THREADS) k_merge(const Op op) {
  const int lane = threadIdx.x & 31;
  const i64 j = (i64)blockIdx.x * DGNN_WARPS + (threadIdx.x >> 5);
  const i64 cs = j * DGNN_SEG;
  if (cs >= op.nnz) return;
  const i64 ce = (cs + DGNN_SEG < op.nnz) ? cs + DGNN_SEG : op.nnz;
  const i64 r = find_row(op.indptr, op.idx_bits, op.n_rows, ce - 1);
  const i64 lb = ldp(op.indptr, op.idx_bits, r);
  const i64 hb = ldp(op.indptr, op.idx_bits, r + 1);
  if (hb - lb <= DGNN_SEG || lb < cs) return;  // the long row that begins in this chunk
  bool first, last;
  if (!dgnn_row_role(op, r, first, last)) return;   // a row this long has entries in this stage; kept for symmetry
  typename Op::State st;
  op.init(st, r, lane);
  op.resume(st, r, lane, first);
  op.merge_partial(st, op.ws + (2 * j + 1) * op.slot_stride, lane);
  for (i64 jj = j + 1; jj * DGNN_SEG < hb; ++jj) op.merge_partial(st, op.ws + (2 * jj) * op.slot_stride, lane);
  op.finalize(st, r, lane, last);
}

static inline unsigned dgnn_grid(i64 items, int per_block) {
  i64 g = (items + per_block - 1) / per_block;
  return (unsigned)(g < 1 ? 1 : g);
}
static inline i64 dgnn_num_chunks(i64 nnz) { return (nnz + DGNN_SEG - 1) / DGNN_SEG; }

// Launch the row / chunk / merge trio for one operator.  `counter` points at 16
// zero-able bytes of workspace (the two row counters of k_rows).
// kernels whose dynamic shared memory exceeds the 48 KB default need the limit raised once per launch site
template <class K>
static inline cudaError_t dgnn_allow_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <class Op>
static inline int dgnn_launch_trio(const Op& op, unsigned long long* counter, cudaStream_t s) {
  if (op.n_rows <= 0) return DGNN_OK;
  const size_t ring = (size_t)op.ring_bytes();          // staging area per warp (0 for operators that gather into registers)
  const size_t row_smem = ring * DGNN_ROW_WARPS;
  cudaError_t e;
  if (op.nnz <= DGNN_SMALL_NNZ) {
    if ((e = dgnn_allow_smem(k_rows_small<Op>, row_smem)) != cudaSuccess) return (int)e;
    k_rows_small<Op><<<dgnn_grid(op.n_rows, DGNN_ROW_WARPS), DGNN_ROW_THREADS, row_smem, s>>>(op);
    cudaError_t e0 = cudaGetLastError();
    return e0 == cudaSuccess ? DGNN_OK : (int)e0;
  }
  e = cudaMemsetAsync(counter, 0, 2 * sizeof(unsigned long long), s);
  if (e != cudaSuccess) return (int)e;
  {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int per_sm = Op::MIN_BLOCKS;                         // resident CTAs per SM: registers, or the staging areas
    if (row_smem > 0) {
      const int fit = (int)((227 * 1024) / (row_smem + 1024));
      if (fit < per_sm) per_sm = fit < 1 ? 1 : fit;
    }
    const i64 pool = (i64)sms * per_sm;                  // one wave, rows are drawn dynamically
    const i64 need = (op.n_rows + DGNN_ROW_WARPS - 1) / DGNN_ROW_WARPS;
    // rows per draw: about 64 edges' worth, one row once the average row has 32 edges or more
    const i64 avg = op.nnz / op.n_rows;
    int batch = avg >= 32 ? 1 : (int)(64 / (avg > 2 ? avg : 2));
    if (batch > 31) batch = 31;  // the batch's pointers plus one fit the 32 lanes
    if ((e = dgnn_allow_smem(k_rows<Op>, row_smem)) != cudaSuccess) return (int)e;
    k_rows<Op><<<(unsigned)(need < pool ? need : pool), DGNN_ROW_THREADS, row_smem, s>>>(op, counter, batch);
  }
  if (op.nnz > DGNN_SEG) {
    const i64 nc = dgnn_num_chunks(op.nnz);
    const size_t part = Op::HAS_PARTIALS ? (((size_t)(DGNN_CHUNK_WARPS - 1) * op.slot_stride + 3) / 4) * 16 : 0;
    const size_t smem = part + ring * DGNN_CHUNK_WARPS;
    if ((e = dgnn_allow_smem(k_chunks<Op>, smem)) != cudaSuccess) return (int)e;
    k_chunks<Op><<<(unsigned)(2 * nc), DGNN_CHUNK_WARPS * 32, smem, s>>>(op);
    if (Op::HAS_PARTIALS) k_merge<Op><<<dgnn_grid(nc, DGNN_WARPS), DGNN_THREADS, 0, s>>>(op);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

// workspaces start with this many bytes reserved for the row counter
constexpr size_t DGNN_WS_HEADER = 256;

static inline int ilog2_exact(int x) {  // -1 unless x is a power of two
  if (x <= 0 || (x & (x - 1))) return -1;
  int s = 0;
  while ((1 << s) < x) ++s;
  return s;
}

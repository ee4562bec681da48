// Attention-logit kernels of the GAT layer, fused around the aggregation operator.
//
// The reference layer computes attn_row = (attn_l * h).sum(-1) and
// attn_col = (attn_r * h).sum(-1) with separate elementwise and reduction passes
// over the [N,H,F] projected features (layers/gatconv_layer.py:74-75), and autograd
// adds three more full-size passes in the backward.  Here one streaming pass
// produces both logits, and one streaming pass of the backward adds
//   grad_h += grad_row (x) attn_l + grad_col (x) attn_r        (in place)
// and accumulates grad_attn_l / grad_attn_r.  A warp owns whole rows (lane l holds
// float4 vectors l, l+32, ... exactly as in the aggregation kernels), so the
// column a lane accumulates never changes and the parameter gradients stay in
// registers until one fixed-order fold per CTA and one over CTAs.
#include "common.cuh"

namespace {

constexpr int LG_WARPS = 8;
constexpr int LG_THREADS = LG_WARPS * 32;

struct Shape {
  bool ok;
  int hf4, f4_shift, vpl;
};
inline Shape shape_of(int h, int f) {
  Shape s{false, 0, 0, 0};
  if (f % 4) return s;
  const int sh = ilog2_exact(f / 4);
  if (sh < 0) return s;
  const i64 hf4 = (i64)h * (f / 4);
  if (hf4 > 256) return s;
  s.ok = true; s.hf4 = (int)hf4; s.f4_shift = sh;
  s.vpl = hf4 <= 32 ? 1 : hf4 <= 64 ? 2 : hf4 <= 128 ? 4 : 8;
  return s;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline size_t up256(size_t x) { return (x + 255) & ~size_t(255); }

// Fan-out of a rank's rows into its send buffer (sharded layer): row r is copied to the send-buffer rows
// pos[ptr[r]] .. pos[ptr[r+1]-1], one per (peer, chunk) that fetches it.  ptr == NULL: no fan-out.
struct LogitsFan {
  const int* ptr;
  const int* pos;
  float4* feat;      // [send rows, hf4]
  float* attn_col;   // [send rows, H]
};

template <int VPL>
__global__ void __launch_bounds__(LG_THREADS)
k_logits_fwd(i64 n, int H, int hf4, int f4_shift, const float4* feat, const float4* al, const float4* ar,
             float* attn_row, float* attn_col, const LogitsFan fan) {
  const int lane = threadIdx.x & 31;
  LaneMap<VPL> lm;
  lm.init(lane, hf4, f4_shift);
  float4 l4[VPL], r4[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    l4[v] = lm.act[v] ? ld4(al + lm.q[v]) : zero4();
    r4[v] = lm.act[v] ? ld4(ar + lm.q[v]) : zero4();
  }
  const i64 stride = (i64)gridDim.x * LG_WARPS;
  // two rows per iteration: twice the loads in flight per warp
  for (i64 r = (i64)blockIdx.x * LG_WARPS + (threadIdx.x >> 5); r < n; r += 2 * stride) {
    const i64 r2 = r + stride;
    const bool two = r2 < n;
    float4 xa[VPL], xb[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      xa[v] = lm.act[v] ? ld4(feat + r * hf4 + lm.q[v]) : zero4();
      xb[v] = (two && lm.act[v]) ? ld4(feat + r2 * hf4 + lm.q[v]) : zero4();
    }
    float d[4][VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      d[0][v] = dot4(xa[v], l4[v]);
      d[1][v] = dot4(xa[v], r4[v]);
      d[2][v] = dot4(xb[v], l4[v]);
      d[3][v] = dot4(xb[v], r4[v]);
    }
    head_reduce<4, VPL>(d, f4_shift);
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (lm.lead[v]) {
        attn_row[r * H + lm.hd[v]] = d[0][v];
        attn_col[r * H + lm.hd[v]] = d[1][v];
        if (two) {
          attn_row[r2 * H + lm.hd[v]] = d[2][v];
          attn_col[r2 * H + lm.hd[v]] = d[3][v];
        }
      }
    }
    if (fan.ptr) {   // the row is in registers: write the copies its fetchers will read
      for (int k = 0; k < (two ? 2 : 1); ++k) {
        const i64 rr = k ? r2 : r;
        const int lo = __ldg(fan.ptr + rr), hi = __ldg(fan.ptr + rr + 1);
        for (int j = lo; j < hi; ++j) {
          const i64 p = __ldg(fan.pos + j);
#pragma unroll
          for (int v = 0; v < VPL; ++v) {
            if (!lm.act[v]) continue;
            fan.feat[p * hf4 + lm.q[v]] = k ? xb[v] : xa[v];
            if (lm.lead[v]) fan.attn_col[p * H + lm.hd[v]] = k ? d[3][v] : d[1][v];
          }
        }
      }
    }
  }
}

// part layout: [cta][2][hf4] float4  (0: grad_attn_l, 1: grad_attn_r)
template <int VPL>
__global__ void __launch_bounds__(LG_THREADS)
k_logits_bwd(i64 n, int H, int hf4, int f4_shift, const float4* feat, const float4* al, const float4* ar,
             const float* grad_row, const float* grad_col, float4* grad_feat, float4* part) {
  extern __shared__ float4 sm4[];   // [LG_WARPS][2][hf4]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  LaneMap<VPL> lm;
  lm.init(lane, hf4, f4_shift);
  float4 l4[VPL], r4[VPL], accl[VPL], accr[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    l4[v] = lm.act[v] ? ld4(al + lm.q[v]) : zero4();
    r4[v] = lm.act[v] ? ld4(ar + lm.q[v]) : zero4();
    accl[v] = zero4();
    accr[v] = zero4();
  }
  const i64 stride = (i64)gridDim.x * LG_WARPS;
  for (i64 r = (i64)blockIdx.x * LG_WARPS + warp; r < n; r += stride) {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (!lm.act[v]) continue;
      const float gr = __ldg(grad_row + r * H + lm.hd[v]);
      const float gc = __ldg(grad_col + r * H + lm.hd[v]);
      const float4 x = ld4(feat + r * hf4 + lm.q[v]);
      float4 g = grad_feat[r * hf4 + lm.q[v]];
      fma4(g, gr, l4[v]);
      fma4(g, gc, r4[v]);
      grad_feat[r * hf4 + lm.q[v]] = g;
      fma4(accl[v], gr, x);
      fma4(accr[v], gc, x);
    }
  }
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    if (!lm.act[v]) continue;
    sm4[(warp * 2 + 0) * hf4 + lm.q[v]] = accl[v];
    sm4[(warp * 2 + 1) * hf4 + lm.q[v]] = accr[v];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * hf4; i += LG_THREADS) {
    float4 s = zero4();
    for (int w = 0; w < LG_WARPS; ++w) add4(s, sm4[w * 2 * hf4 + i]);   // fixed warp order
    part[(i64)blockIdx.x * 2 * hf4 + i] = s;
  }
}

__global__ void k_logits_bwd_final(int ctas, int hf4, const float4* part, float4* grad_l, float4* grad_r) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * hf4) return;
  float4 s = zero4();
  for (int c = 0; c < ctas; ++c) add4(s, part[(i64)c * 2 * hf4 + i]);     // fixed CTA order
  if (i < hf4) grad_l[i] = s; else grad_r[i - hf4] = s;
}

inline int bwd_ctas() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms * 4;
}

}  // namespace

extern "C" {

int dgnn_gat_logits_forward(int64_t n, int h, int f, const float* feat, const float* attn_l, const float* attn_r,
                            float* attn_row, float* attn_col, void* stream) {
  return dgnn_gat_logits_forward_fan(n, h, f, feat, attn_l, attn_r, attn_row, attn_col, nullptr, nullptr, nullptr, nullptr,
                                     stream);
}

int dgnn_gat_logits_forward_fan(int64_t n, int h, int f, const float* feat, const float* attn_l, const float* attn_r,
                                float* attn_row, float* attn_col, const int32_t* send_ptr, const int32_t* send_pos,
                                float* send_feat, float* send_attn_col, void* stream) {
  if (n < 0 || h <= 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (n == 0) return DGNN_OK;
  if (!feat || !attn_l || !attn_r || !attn_row || !attn_col) return DGNN_ERR_NULL;
  if (send_ptr && (!send_pos || !send_feat || !send_attn_col)) return DGNN_ERR_NULL;
  if (send_ptr && !aligned16(send_feat)) return DGNN_ERR_ALIGN;
  const LogitsFan fan{send_ptr, send_pos, reinterpret_cast<float4*>(send_feat), send_attn_col};
  const Shape sp = shape_of(h, f);
  if (!sp.ok) return DGNN_ERR_SHAPE;   // callers fall back to separate tensor ops for other shapes
  if (!aligned16(feat) || !aligned16(attn_l) || !aligned16(attn_r)) return DGNN_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const i64 need = (n + LG_WARPS - 1) / LG_WARPS;
  const unsigned grid = (unsigned)(need < (i64)bwd_ctas() * 2 ? need : (i64)bwd_ctas() * 2);
  const float4* x = reinterpret_cast<const float4*>(feat);
  const float4* l = reinterpret_cast<const float4*>(attn_l);
  const float4* r = reinterpret_cast<const float4*>(attn_r);
  switch (sp.vpl) {
    case 1: k_logits_fwd<1><<<grid, LG_THREADS, 0, s>>>(n, h, sp.hf4, sp.f4_shift, x, l, r, attn_row, attn_col, fan); break;
    case 2: k_logits_fwd<2><<<grid, LG_THREADS, 0, s>>>(n, h, sp.hf4, sp.f4_shift, x, l, r, attn_row, attn_col, fan); break;
    case 4: k_logits_fwd<4><<<grid, LG_THREADS, 0, s>>>(n, h, sp.hf4, sp.f4_shift, x, l, r, attn_row, attn_col, fan); break;
    default: k_logits_fwd<8><<<grid, LG_THREADS, 0, s>>>(n, h, sp.hf4, sp.f4_shift, x, l, r, attn_row, attn_col, fan); break;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

size_t dgnn_gat_logits_backward_workspace_bytes(int h, int f) {
  if (h <= 0 || f <= 0) return 256;
  return up256((size_t)148 * 8 * 2 * h * f * sizeof(float)) + 256;   // room for up to 1184 CTAs
}

int dgnn_gat_logits_backward(int64_t n, int h, int f, const float* feat, const float* attn_l, const float* attn_r,
                             const float* grad_row, const float* grad_col, float* grad_feat, float* grad_l,
                             float* grad_r, void* workspace, size_t workspace_bytes, void* stream) {
  if (n < 0 || h <= 0 || f <= 0) return DGNN_ERR_SHAPE;
  if (!attn_l || !attn_r || !grad_l || !grad_r) return DGNN_ERR_NULL;
  if (n > 0 && (!feat || !grad_row || !grad_col || !grad_feat)) return DGNN_ERR_NULL;
  const Shape sp = shape_of(h, f);
  if (!sp.ok) return DGNN_ERR_SHAPE;
  if (!aligned16(feat) || !aligned16(attn_l) || !aligned16(attn_r) || !aligned16(grad_feat) || !aligned16(grad_l) ||
      !aligned16(grad_r))
    return DGNN_ERR_ALIGN;
  if (!workspace || workspace_bytes < dgnn_gat_logits_backward_workspace_bytes(h, f)) return DGNN_ERR_WORKSPACE;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float4* part = reinterpret_cast<float4*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  const i64 need = (n + LG_WARPS - 1) / LG_WARPS;
  int ctas = bwd_ctas();
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (need < ctas) ctas = (int)(need < 1 ? 1 : need);
  const size_t smem = (size_t)LG_WARPS * 2 * sp.hf4 * sizeof(float4);   // <= 64 KB at hf4 = 256
  const float4* x = reinterpret_cast<const float4*>(feat);
  const float4* l = reinterpret_cast<const float4*>(attn_l);
  const float4* r = reinterpret_cast<const float4*>(attn_r);
  float4* g = reinterpret_cast<float4*>(grad_feat);
#define LG_BWD(V)                                                                                               \
  {                                                                                                             \
    if (smem > 48 * 1024)                                                                                       \
      cudaFuncSetAttribute(k_logits_bwd<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    k_logits_bwd<V><<<ctas, LG_THREADS, smem, s>>>(n, h, sp.hf4, sp.f4_shift, x, l, r, grad_row, grad_col, g, part); \
  }
  switch (sp.vpl) {
    case 1: LG_BWD(1) break;
    case 2: LG_BWD(2) break;
    case 4: LG_BWD(4) break;
    default: LG_BWD(8) break;
  }
#undef LG_BWD
  k_logits_bwd_final<<<dgnn_grid(2 * sp.hf4, 128), 128, 0, s>>>(ctas, sp.hf4, part, reinterpret_cast<float4*>(grad_l),
                                                              reinterpret_cast<float4*>(grad_r));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? DGNN_OK : (int)e;
}

}  // extern "C"

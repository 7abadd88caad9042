// Sequence-mixer kernels over a packed (unpadded) batch: grouped / gated RMS norm, paged key / value write, windowed
// attention with kept first tokens and a softmax sink, causal depthwise convolution with carried taps, linear attention
// with a fixed decay, and the gated delta rule. Statistics, scores, decays and recurrent state are fp32; tensors are read
// and written as fp32 or bf16 according to their dtype arguments. Every kernel takes the batch as (cu_tokens, pos0, slot)
// device arrays, so one launch serves sequences that start, continue or advance by one token, and nothing depends on where
// a sequence sits in the batch.
#include <math.h>

#include "seqmix.cuh"

namespace vy {

// ---- RMS norm -------------------------------------------------------------------------------------------------------
struct NormDev {
  long long rows; int groups, width;
  const int* row_index;
  const void* x; long long ldx; int x_dt;
  const void* w; int w_dt, w_mode, w_full;   // w_full: the weight covers the whole row (one entry per element), not one group
  const void* gate; long long ld_gate; int gate_dt, gate_act;
  float eps, coef; int accumulate;
  void* out; long long ld_out; int out_dt;
  void* copy; long long ld_copy; int copy_dt;
};

__global__ void __launch_bounds__(128) rms_norm_kernel(NormDev d) {
  pdl_trigger();
  pdl_wait();
  const long long r = blockIdx.x * 4LL + (threadIdx.x >> 5);
  if (r >= d.rows) return;
  const int lane = threadIdx.x & 31;
  const long long tok = r / d.groups;
  const int grp = static_cast<int>(r - tok * d.groups);
  const long long st = d.row_index ? d.row_index[tok] : tok;
  const long long xo = st * d.ldx + static_cast<long long>(grp) * d.width;
  float ss = 0.f;
  for (int c = lane; c < d.width; c += 32) {
    const float v = ld_as_float(d.x, d.x_dt, xo + c);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = d.coef / sqrtf(ss / static_cast<float>(d.width) + d.eps);
  const long long go = st * d.ld_gate + static_cast<long long>(grp) * d.width;
  const long long oo = tok * d.ld_out + static_cast<long long>(grp) * d.width;
  const int wo = d.w_full ? grp * d.width : 0;
  for (int c = lane; c < d.width; c += 32) {
    float y = ld_as_float(d.x, d.x_dt, xo + c) * inv;
    if (d.w_mode == 1) y *= ld_as_float(d.w, d.w_dt, wo + c);
    else if (d.w_mode == 2) y *= 1.f + ld_as_float(d.w, d.w_dt, wo + c);
    if (d.gate) y *= apply_uact(ld_as_float(d.gate, d.gate_dt, go + c), d.gate_act);
    if (d.accumulate) y += ld_as_float(d.out, d.out_dt, oo + c);
    st_from_float(d.out, d.out_dt, oo + c, y);
    if (d.copy) st_from_float(d.copy, d.copy_dt, tok * d.ld_copy + static_cast<long long>(grp) * d.width + c, y);
  }
}

// The same with the row held in registers (one read of x) and TPR threads per row, 256 threads per CTA: for widths up to
// 8 TPR. Few wide rows (single-token steps) get many threads each; many narrow rows get a warp each.
// VEC: x, gate and out rows start on 16-byte boundaries (out: 8 when bf16) and the width is a multiple of 4, x and gate are fp32,
// and an accumulating call's out is fp32: each thread then moves two groups of 4 adjacent elements instead of 8 strided ones,
// a quarter of the load / store / address instructions (a single-token call is one short dependent instruction stream per warp)
template <int TPR, bool VEC>
__global__ void __launch_bounds__(256) rms_norm_cached_kernel(NormDev d) {
  pdl_trigger();
  pdl_wait();
  constexpr int NC = 8, RPB = 256 / TPR;
  __shared__ float part[RPB][TPR / 32 + 1];
  const int lr = threadIdx.x / TPR, lt = threadIdx.x % TPR;
  const unsigned r = blockIdx.x * static_cast<unsigned>(RPB) + lr;   // the launcher keeps rows below 2^31: 32-bit division
  const bool live = r < static_cast<unsigned>(d.rows);
  const unsigned tok = live ? (d.groups == 1 ? r : r / static_cast<unsigned>(d.groups)) : 0u;
  const int grp = live ? static_cast<int>(r - tok * static_cast<unsigned>(d.groups)) : 0;
  const long long st = d.row_index ? d.row_index[tok] : static_cast<long long>(tok);
  const long long xo = st * d.ldx + static_cast<long long>(grp) * d.width;
  float xv[NC];
  float ss = 0.f;
  if constexpr (VEC) {
    const float* xp = reinterpret_cast<const float*>(d.x) + xo;
#pragma unroll
    for (int i = 0; i < NC / 4; ++i) {
      const int c = 4 * lt + i * 4 * TPR;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live && c < d.width) v = *reinterpret_cast<const float4*>(xp + c);
      xv[4 * i] = v.x; xv[4 * i + 1] = v.y; xv[4 * i + 2] = v.z; xv[4 * i + 3] = v.w;
    }
#pragma unroll
    for (int i = 0; i < NC; ++i) ss = fmaf(xv[i], xv[i], ss);
  } else {
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int c = lt + i * TPR;
      xv[i] = (live && c < d.width) ? ld_as_float(d.x, d.x_dt, xo + c) : 0.f;
      ss = fmaf(xv[i], xv[i], ss);
    }
  }
  ss = warp_sum(ss);
  if (TPR > 32) {
    if ((threadIdx.x & 31) == 0) part[lr][lt >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int w = 0; w < TPR / 32; ++w) ss += part[lr][w];
  }
  if (!live) return;
  const float inv = d.coef / sqrtf(ss / static_cast<float>(d.width) + d.eps);
  const int wo = d.w_full ? grp * d.width : 0;
  if constexpr (VEC) {
    const long long go = st * d.ld_gate + static_cast<long long>(grp) * d.width;
    const long long oo = static_cast<long long>(tok) * d.ld_out + static_cast<long long>(grp) * d.width;
#pragma unroll
    for (int i = 0; i < NC / 4; ++i) {
      const int c = 4 * lt + i * 4 * TPR;
      if (c >= d.width) continue;
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        y[e] = xv[4 * i + e] * inv;
        if (d.w_mode == 1) y[e] *= ld_as_float(d.w, d.w_dt, wo + c + e);
        else if (d.w_mode == 2) y[e] *= 1.f + ld_as_float(d.w, d.w_dt, wo + c + e);
      }
      if (d.gate) {
        const float4 g = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(d.gate) + go + c);
        y[0] *= apply_uact(g.x, d.gate_act); y[1] *= apply_uact(g.y, d.gate_act);
        y[2] *= apply_uact(g.z, d.gate_act); y[3] *= apply_uact(g.w, d.gate_act);
      }
      if (d.out_dt == VY_F32) {
        float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(d.out) + oo + c);
        if (d.accumulate) {
          const float4 o = *op;
          y[0] += o.x; y[1] += o.y; y[2] += o.z; y[3] += o.w;
        }
        *op = make_float4(y[0], y[1], y[2], y[3]);
        if (d.copy) {
          const long long co = static_cast<long long>(tok) * d.ld_copy + static_cast<long long>(grp) * d.width + c;
#pragma unroll
          for (int e = 0; e < 4; ++e) st_from_float(d.copy, d.copy_dt, co + e, y[e]);
        }
      } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
        uint2 pk;
        pk.x = *reinterpret_cast<const unsigned*>(&lo);
        pk.y = *reinterpret_cast<const unsigned*>(&hi);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(d.out) + oo + c) = pk;
      }
    }
    return;
  }
  const long long go = st * d.ld_gate + static_cast<long long>(grp) * d.width;
  const long long oo = static_cast<long long>(tok) * d.ld_out + static_cast<long long>(grp) * d.width;
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    const int c = lt + i * TPR;
    if (c < d.width) {
      float y = xv[i] * inv;
      if (d.w_mode == 1) y *= ld_as_float(d.w, d.w_dt, wo + c);
      else if (d.w_mode == 2) y *= 1.f + ld_as_float(d.w, d.w_dt, wo + c);
      if (d.gate) y *= apply_uact(ld_as_float(d.gate, d.gate_dt, go + c), d.gate_act);
      if (d.accumulate) y += ld_as_float(d.out, d.out_dt, oo + c);
      st_from_float(d.out, d.out_dt, oo + c, y);
      if (d.copy) st_from_float(d.copy, d.copy_dt, static_cast<long long>(tok) * d.ld_copy + static_cast<long long>(grp) * d.width + c, y);
    }
  }
}

// ---- paged key / value write ------------------------------------------------------------------------------------------
struct KvwDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  const void* k; long long ldk; const void* v; long long ldv; int in_dt;
  int kw, vw;
  void* kp; void* vp; int pool_dt;
};

__global__ void __launch_bounds__(128) kv_page_write_kernel(KvwDev d) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int pos = d.pos0[s] + i;
    const long long row = static_cast<long long>(d.table[static_cast<long long>(s) * d.tw + pos / d.bs]) * d.bs + pos % d.bs;
    const long long src = base + i;
    for (int c = threadIdx.x; c < d.kw + d.vw; c += blockDim.x) {
      if (c < d.kw) st_from_float(d.kp, d.pool_dt, row * d.kw + c, ld_as_float(d.k, d.in_dt, src * d.ldk + c));
      else st_from_float(d.vp, d.pool_dt, row * d.vw + (c - d.kw), ld_as_float(d.v, d.in_dt, src * d.ldv + (c - d.kw)));
    }
  }
}

// ---- windowed attention with kept first tokens and a sink ---------------------------------------------------------------

constexpr int WA_WARPS = 4;
constexpr int WA_VR = 8;  // value columns per lane: vdim <= 256
constexpr int WA_TILED_MIN = 16;   // longest portion of a step from which the tiled prompt kernel (seqmix_tiled.cu) takes over
constexpr int LA_CHUNKED_MIN = 8;  // same for the chunked linear attention

__device__ __forceinline__ float dot_row(const void* base, int dt, long long off, int n, const float* __restrict__ qs) {
  float acc = 0.f;
  if (dt == VY_F32 && (n & 3) == 0 && (off & 3) == 0) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    for (int i = 0; i < (n >> 2); ++i) {
      const float4 k = p[i];
      acc = fmaf(qs[4 * i], k.x, acc);
      acc = fmaf(qs[4 * i + 1], k.y, acc);
      acc = fmaf(qs[4 * i + 2], k.z, acc);
      acc = fmaf(qs[4 * i + 3], k.w, acc);
    }
  } else if (dt == VY_BF16 && (n & 7) == 0 && (off & 7) == 0) {
    for (int i = 0; i < n; i += 8) {
      float k[8];
      ld8_as_float(base, dt, off + i, k);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(qs[i + j], k[j], acc);
    }
  } else {
    for (int i = 0; i < n; ++i) acc = fmaf(qs[i], ld_as_float(base, dt, off + i), acc);
  }
  return acc;
}

// portions of a few tokens: one warp per query, lanes over 32 keys at a time
__global__ void __launch_bounds__(WA_WARPS * 32) window_attn_kernel(WinDev d) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float wa_smem[];
  const int s = blockIdx.z, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  const int qi = static_cast<int>(blockIdx.x) * WA_WARPS + warp;
  if (qi >= n) return;  // the warps never meet at a CTA barrier
  const int g = h / (d.heads / d.kv_heads);
  float* qs = wa_smem + warp * d.dim;
  const long long qrow = base + qi;
  for (int i = lane; i < d.dim; i += 32) qs[i] = ld_as_float(d.q, d.q_dt, qrow * d.ldq + static_cast<long long>(h) * d.dim + i);
  __syncwarp();
  const int pos = d.pos0[s] + qi;
  // visible keys: [0, nA) (kept first tokens) and [lowB, pos] (the window), disjoint by construction
  int nA, lowB;
  visible_keys(d, pos, nA, lowB);
  const int count = nA + (pos + 1 - lowB);
  float m = -INFINITY, l = 0.f;
  if (d.sink) {
    m = ld_as_float(d.sink, d.sink_dt, h);
    l = 1.f;
  }
  float acc[WA_VR];
#pragma unroll
  for (int r = 0; r < WA_VR; ++r) acc[r] = 0.f;
  const int* tab = d.table + static_cast<long long>(s) * d.tw;
  const long long kstride = d.k_row, vstride = d.v_row;
  const int tiles = (count + 31) >> 5;
  for (int tt = 0; tt < tiles; ++tt) {
    const int c = tt * 32 + lane;
    const bool valid = c < count;
    long long row = 0;
    float sc = -INFINITY;
    if (valid) {
      const int kp = c < nA ? c : lowB + (c - nA);
      row = static_cast<long long>(tab[kp / d.bs]) * d.bs + kp % d.bs;
      sc = dot_row(d.kp, d.pool_dt, row * kstride + static_cast<long long>(g) * d.dim, d.dim, qs) * d.scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float p = valid ? expf(sc - m_new) : 0.f;
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int r = 0; r < WA_VR; ++r) acc[r] *= corr;
    const int nv = min(32, count - tt * 32);
    for (int jj = 0; jj < nv; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long rj = __shfl_sync(0xffffffffu, row, jj);
      const long long vo = rj * vstride + static_cast<long long>(g) * d.vdim;
#pragma unroll
      for (int r = 0; r < WA_VR; ++r) {
        const int col = lane + 32 * r;
        if (col < d.vdim) acc[r] = fmaf(pj, ld_as_float(d.vp, d.pool_dt, vo + col), acc[r]);
      }
    }
  }
  float og = d.out_scale / l;
  if (d.gate) og *= sigmoidf_(ld_as_float(d.gate, d.gate_dt, qrow * d.ld_gate + h));
#pragma unroll
  for (int r = 0; r < WA_VR; ++r) {
    const int col = lane + 32 * r;
    if (col < d.vdim) st_from_float(d.out, d.out_dt, qrow * d.ld_out + static_cast<long long>(h) * d.vdim + col, acc[r] * og);
  }
}

// single tokens: one CTA per (head, sequence); its warps take the visible keys four at a time, round-robin, each lane holding
// every 32nd channel of the query and of the output (coalesced key / value rows), and the warps' partial softmaxes are merged
// in warp order at the end
constexpr int WD_WARPS = 8;
constexpr int WD_KEYS = 4;

// VEC: fp32 pages and query, dim and vdim multiples of 4, 16-byte aligned rows: lane l holds channels 4 l .. 4 l + 3 (+ 128) and
// reads a key or value row with one 16-byte load per 128 channels instead of four 4-byte ones.
// HG: query heads per CTA, all reading the same key / value head (grouped heads; the single head of latent rows): a key or value
// row is loaded once and used by the HG heads, so the pages cross L2 heads / HG times instead of heads times
template <bool VEC, int HG>
__global__ void __launch_bounds__(WD_WARPS * 32) window_attn_decode_kernel(WinDev d) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float wa_smem[];
  const int s = blockIdx.z, h0 = blockIdx.y * HG;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = d.cu[s];
  if (d.cu[s + 1] - base <= 0) return;
  const int g = h0 / (d.heads / d.kv_heads);
  const long long qrow = base;
  // channel of register slot r: strided by 32 (scalar form) or groups of 4 strided by 128 (vector form)
  auto chan = [&](int r) { return VEC ? 4 * lane + 128 * (r >> 2) + (r & 3) : lane + 32 * r; };
  float qreg[HG][WA_VR];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh)
#pragma unroll
    for (int r = 0; r < WA_VR; ++r) {
      const int col = chan(r);
      qreg[hh][r] = col < d.dim ? ld_as_float(d.q, d.q_dt, qrow * d.ldq + static_cast<long long>(h0 + hh) * d.dim + col) * d.scale : 0.f;
    }
  const int pos = d.pos0[s];
  int nA, lowB;
  visible_keys(d, pos, nA, lowB);
  const int count = nA + (pos + 1 - lowB);
  float m[HG], l[HG];
  float acc[HG][WA_VR];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    m[hh] = -INFINITY;
    l[hh] = 0.f;
    if (d.sink && warp == 0) {
      m[hh] = ld_as_float(d.sink, d.sink_dt, h0 + hh);
      l[hh] = 1.f;
    }
#pragma unroll
    for (int r = 0; r < WA_VR; ++r) acc[hh][r] = 0.f;
  }
  const int* tab = d.table + static_cast<long long>(s) * d.tw;
  const long long kstride = d.k_row, vstride = d.v_row;
  for (int c0 = WD_KEYS * warp; c0 < count; c0 += WD_KEYS * WD_WARPS) {
    long long row[WD_KEYS];
    float sc[HG][WD_KEYS], vv[WD_KEYS][WA_VR];
#pragma unroll
    for (int u = 0; u < WD_KEYS; ++u) {
      const int c = min(c0 + u, count - 1);   // past the end: a repeat of the last key, given weight 0 below
      const int kp = c < nA ? c : lowB + (c - nA);
      row[u] = static_cast<long long>(tab[kp / d.bs]) * d.bs + kp % d.bs;
#pragma unroll
      for (int hh = 0; hh < HG; ++hh) sc[hh][u] = 0.f;
    }
    if constexpr (VEC) {
      const float* kb = reinterpret_cast<const float*>(d.kp) + static_cast<long long>(g) * d.dim + 4 * lane;
      const float* vb = reinterpret_cast<const float*>(d.vp) + static_cast<long long>(g) * d.vdim + 4 * lane;
#pragma unroll
      for (int r4 = 0; r4 < WA_VR / 4; ++r4) {
        if (4 * lane + 128 * r4 < d.dim) {
#pragma unroll
          for (int u = 0; u < WD_KEYS; ++u) {
            const float4 k4 = *reinterpret_cast<const float4*>(kb + row[u] * kstride + 128 * r4);
#pragma unroll
            for (int hh = 0; hh < HG; ++hh) {
              sc[hh][u] = fmaf(qreg[hh][4 * r4], k4.x, sc[hh][u]);
              sc[hh][u] = fmaf(qreg[hh][4 * r4 + 1], k4.y, sc[hh][u]);
              sc[hh][u] = fmaf(qreg[hh][4 * r4 + 2], k4.z, sc[hh][u]);
              sc[hh][u] = fmaf(qreg[hh][4 * r4 + 3], k4.w, sc[hh][u]);
            }
          }
        }
      }
#pragma unroll
      for (int r4 = 0; r4 < WA_VR / 4; ++r4) {
#pragma unroll
        for (int u = 0; u < WD_KEYS; ++u) {
          float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (4 * lane + 128 * r4 < d.vdim) v4 = *reinterpret_cast<const float4*>(vb + row[u] * vstride + 128 * r4);
          vv[u][4 * r4] = v4.x; vv[u][4 * r4 + 1] = v4.y; vv[u][4 * r4 + 2] = v4.z; vv[u][4 * r4 + 3] = v4.w;
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < WA_VR; ++r) {
        const int col = lane + 32 * r;
        if (col < d.dim) {
#pragma unroll
          for (int u = 0; u < WD_KEYS; ++u) {
            const float kv = ld_as_float(d.kp, d.pool_dt, row[u] * kstride + static_cast<long long>(g) * d.dim + col);
#pragma unroll
            for (int hh = 0; hh < HG; ++hh) sc[hh][u] = fmaf(qreg[hh][r], kv, sc[hh][u]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < WA_VR; ++r) {
        const int col = lane + 32 * r;
#pragma unroll
        for (int u = 0; u < WD_KEYS; ++u)
          vv[u][r] = col < d.vdim ? ld_as_float(d.vp, d.pool_dt, row[u] * vstride + static_cast<long long>(g) * d.vdim + col) : 0.f;
      }
    }
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
      float m_new = m[hh];
#pragma unroll
      for (int u = 0; u < WD_KEYS; ++u) {
        sc[hh][u] = c0 + u < count ? warp_sum(sc[hh][u]) : -INFINITY;
        m_new = fmaxf(m_new, sc[hh][u]);
      }
      const float corr = m[hh] == -INFINITY ? 0.f : expf(m[hh] - m_new);
      float p[WD_KEYS], ps = 0.f;
#pragma unroll
      for (int u = 0; u < WD_KEYS; ++u) {
        p[u] = c0 + u < count ? expf(sc[hh][u] - m_new) : 0.f;
        ps += p[u];
      }
      l[hh] = fmaf(l[hh], corr, ps);
      m[hh] = m_new;
#pragma unroll
      for (int r = 0; r < WA_VR; ++r) {
        float a = acc[hh][r] * corr;
#pragma unroll
        for (int u = 0; u < WD_KEYS; ++u) a = fmaf(p[u], vv[u][r], a);
        acc[hh][r] = a;
      }
    }
  }
  float* ms = wa_smem;                          // [HG][WD_WARPS]
  float* ls = ms + HG * WD_WARPS;               // [HG][WD_WARPS]
  float* as = ls + HG * WD_WARPS;               // [HG][WD_WARPS][vdim]
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    if (lane == 0) { ms[hh * WD_WARPS + warp] = m[hh]; ls[hh * WD_WARPS + warp] = l[hh]; }
#pragma unroll
    for (int r = 0; r < WA_VR; ++r) {
      const int col = chan(r);
      if (col < d.vdim) as[(hh * WD_WARPS + warp) * d.vdim + col] = acc[hh][r];
    }
  }
  __syncthreads();
  if (warp >= HG) return;   // warp w merges head h0 + w (HG <= WD_WARPS)
  const int hh = warp, h = h0 + hh;
  float M = ms[hh * WD_WARPS];
  for (int w = 1; w < WD_WARPS; ++w) M = fmaxf(M, ms[hh * WD_WARPS + w]);
  float lt = 0.f;
  float wgt[WD_WARPS];
#pragma unroll
  for (int w = 0; w < WD_WARPS; ++w) {
    wgt[w] = ms[hh * WD_WARPS + w] == -INFINITY ? 0.f : expf(ms[hh * WD_WARPS + w] - M);
    lt = fmaf(ls[hh * WD_WARPS + w], wgt[w], lt);
  }
  float og = d.out_scale / lt;
  if (d.gate) og *= sigmoidf_(ld_as_float(d.gate, d.gate_dt, qrow * d.ld_gate + h));
#pragma unroll
  for (int r = 0; r < WA_VR; ++r) {
    const int col = chan(r);
    if (col < d.vdim) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < WD_WARPS; ++w) a = fmaf(as[(hh * WD_WARPS + w) * d.vdim + col], wgt[w], a);
      st_from_float(d.out, d.out_dt, qrow * d.ld_out + static_cast<long long>(h) * d.vdim + col, a * og);
    }
  }
}

// ---- causal depthwise convolution with carried taps ------------------------------------------------------------------
struct ConvDev {
  const int* cu; const int* pos0; const int* slot;
  int channels, taps;
  const void* x; long long ldx; int x_dt;
  const void* w; int w_dt;
  float* state;
  int act;
  void* out; long long ld_out; int out_dt;
  int fuse_state;   // every sequence's tokens fit one CTA row: the thread that read a channel's taps also writes the new ones
};
constexpr int CONV_MAX_TAPS = 16;
constexpr int CONV_TOK = 32;

// the last taps - 1 inputs of channel c after the step's n tokens (older ones come from the taps the slot held)
__device__ __forceinline__ void conv_new_taps(const ConvDev& d, int c, int base, int n, bool carried, float* stp) {
  float tmp[CONV_MAX_TAPS];
#pragma unroll
  for (int t = 0; t < CONV_MAX_TAPS - 1; ++t) {
    if (t < d.taps - 1) {
      const int j = n - (d.taps - 1) + t;
      tmp[t] = j >= 0 ? ld_as_float(d.x, d.x_dt, static_cast<long long>(base + j) * d.ldx + c) : (carried ? stp[d.taps - 1 + j] : 0.f);
    }
  }
#pragma unroll
  for (int t = 0; t < CONV_MAX_TAPS - 1; ++t)
    if (t < d.taps - 1) stp[t] = tmp[t];
}

__global__ void __launch_bounds__(128) causal_conv_kernel(ConvDev d) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.z;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (c >= d.channels) return;
  float w[CONV_MAX_TAPS];
#pragma unroll
  for (int t = 0; t < CONV_MAX_TAPS; ++t) w[t] = t < d.taps ? ld_as_float(d.w, d.w_dt, static_cast<long long>(c) * d.taps + t) : 0.f;
  const bool carried = d.pos0[s] > 0;
  const float* stp = d.state + (static_cast<long long>(d.slot[s]) * d.channels + c) * (d.taps - 1);
  for (int i = blockIdx.y * CONV_TOK; i < n && i < (blockIdx.y + 1) * CONV_TOK; ++i) {
    float y = 0.f;
#pragma unroll
    for (int dd = 0; dd < CONV_MAX_TAPS; ++dd) {
      if (dd < d.taps) {
        const int j = i - dd;
        float xv = 0.f;
        if (j >= 0) xv = ld_as_float(d.x, d.x_dt, static_cast<long long>(base + j) * d.ldx + c);
        else if (carried) xv = stp[d.taps - 1 + j];
        y = fmaf(w[d.taps - 1 - dd], xv, y);
      }
    }
    st_from_float(d.out, d.out_dt, static_cast<long long>(base + i) * d.ld_out + c, apply_uact(y, d.act));
  }
  if (d.fuse_state && d.taps > 1 && n > 0)
    conv_new_taps(d, c, base, n, carried, d.state + (static_cast<long long>(d.slot[s]) * d.channels + c) * (d.taps - 1));
}

__global__ void __launch_bounds__(128) causal_conv_state_kernel(ConvDev d) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (c >= d.channels || n <= 0) return;
  conv_new_taps(d, c, base, n, d.pos0[s] > 0, d.state + (static_cast<long long>(d.slot[s]) * d.channels + c) * (d.taps - 1));
}

// ---- recurrences: one thread owns one column of the dim x vdim state in registers ---------------------------------------

template <int DP>
struct RecChunk { static constexpr int CT = DP >= 256 ? 8 : 16; };

// linear attention with a fixed decay: S = decay S + k v^T, o = S^T q
template <int DP>
__global__ void __launch_bounds__(128) linear_attn_kernel(RecDev d) {
  pdl_trigger();
  pdl_wait();
  constexpr int CT = RecChunk<DP>::CT;
  __shared__ float qs[CT][DP];
  __shared__ float ks[CT][DP];
  const int s = blockIdx.z, h = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (n <= 0) return;
  const bool active = j < d.vdim;
  const float decay = d.decay[h];
  float S[DP];
  float* sp = d.state + ((static_cast<long long>(d.slot[s]) * d.heads + h) * d.dim) * d.vdim + j;
  const bool carried = d.pos0[s] > 0;
#pragma unroll
  for (int i = 0; i < DP; ++i) S[i] = (carried && active && i < d.dim) ? sp[static_cast<long long>(i) * d.vdim] : 0.f;
  for (int t0 = 0; t0 < n; t0 += CT) {
    const int nt = min(CT, n - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * DP; e += blockDim.x) {
      const int tt = e / DP, i = e - tt * DP;
      const long long row = base + t0 + tt;
      float qv = 0.f, kv = 0.f;
      if (i < d.dim) {
        qv = apply_uact(ld_as_float(d.q, d.in_dt, row * d.ldq + static_cast<long long>(h) * d.dim + i), d.in_act);
        kv = apply_uact(ld_as_float(d.k, d.in_dt, row * d.ldk + static_cast<long long>(h) * d.dim + i), d.in_act);
      }
      qs[tt][i] = qv;
      ks[tt][i] = kv;
    }
    __syncthreads();
    if (active) {
      for (int tt = 0; tt < nt; ++tt) {
        const long long row = base + t0 + tt;
        const float vj = apply_uact(ld_as_float(d.v, d.in_dt, row * d.ldv + static_cast<long long>(h) * d.vdim + j), d.in_act);
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < DP; ++i) {
          S[i] = fmaf(decay, S[i], ks[tt][i] * vj);
          o = fmaf(S[i], qs[tt][i], o);
        }
        st_from_float(d.out, d.out_dt, row * d.ld_out + static_cast<long long>(h) * d.vdim + j, o);
      }
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < DP; ++i)
      if (i < d.dim) sp[static_cast<long long>(i) * d.vdim] = S[i];
  }
}

// gated delta rule: a column of the state is shared by LANES adjacent lanes, lane `part` holding channels 4 LANES m + 4 part .. + 3
// of every group of 4 LANES (so the chunk's k / q / decay rows are read as one float4 per group, contiguous across the lanes); the
// two contractions over the channels end in log2(LANES) shuffles each. A CTA owns 32 columns: the recurrence is a dependent chain
// per token, so the lanes per column (not the work per lane) set how many warps there are to overlap those chains
template <int DP>
struct DeltaLanes { static constexpr int value = DP >= 32 ? 8 : 4; };

// PLAIN: gated linear attention, the same walk without the correction term (u = v): `a` holds the decays (prepared), q is scaled as read
template <int DP, bool PLAIN>
__global__ void __launch_bounds__(32 * DeltaLanes<DP>::value) delta_rule_kernel(RecDev d) {
  pdl_trigger();
  pdl_wait();
  constexpr int CT = RecChunk<DP>::CT;
  constexpr int LANES = DeltaLanes<DP>::value, T = 32 * LANES;
  constexpr int NM = DP / (4 * LANES);
  extern __shared__ __align__(16) float dr_smem[];
  float (*qs)[DP] = reinterpret_cast<float (*)[DP]>(dr_smem);
  float (*ks)[DP] = reinterpret_cast<float (*)[DP]>(dr_smem + CT * DP);
  float (*gs)[DP] = reinterpret_cast<float (*)[DP]>(dr_smem + 2 * CT * DP);
  float* betas = dr_smem + 3 * CT * DP;
  float* vs = betas + CT;                       // [CT][32]: the chunk's values of this CTA's 32 columns
  const int s = blockIdx.z, h = blockIdx.y;
  const int part = threadIdx.x & (LANES - 1), col = threadIdx.x / LANES;
  const int j = blockIdx.x * 32 + col;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = T >> 5;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (n <= 0) return;
  const bool active = j < d.vdim;
  const int gq = h / (d.heads / d.kv_heads);
  const float neg_rate = PLAIN ? 0.f : -expf(ld_as_float(d.a_log, d.a_log_dt, h));
  const float qscale = 1.f / sqrtf(static_cast<float>(d.dim));
  const float q_in = PLAIN ? d.q_scale : 1.f;
  float S[NM][4];
  float* sp = d.state + ((static_cast<long long>(d.slot[s]) * d.heads + h) * d.dim) * d.vdim + j;
  const bool carried = d.pos0[s] > 0;
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 4 * LANES * m + 4 * part + e;
      S[m][e] = (carried && active && i < d.dim) ? sp[static_cast<long long>(i) * d.vdim] : 0.f;
    }
  // the next chunk's raw q / k / decay inputs travel in registers while the current chunk is walked
  constexpr int NPF = CT * DP / T;
  constexpr int NV = CT * 32 / T;
  float rq[NPF], rk[NPF], ra[NPF], rv[NV], rb = 0.f;
  auto fetch = [&](int t0) {
    const int nt = min(CT, n - t0);
#pragma unroll
    for (int u = 0; u < NPF; ++u) {
      const int e = threadIdx.x + u * T, tt = e / DP, i = e - tt * DP;
      const bool ok = tt < nt && i < d.dim;
      const long long row = base + t0 + tt;
      rq[u] = ok ? ld_as_float(d.q, d.in_dt, row * d.ldq + static_cast<long long>(gq) * d.dim + i) : 0.f;
      rk[u] = ok ? ld_as_float(d.k, d.in_dt, row * d.ldk + static_cast<long long>(gq) * d.dim + i) : 0.f;
      ra[u] = ok ? ld_as_float(d.a, d.a_dt, row * d.ld_a + static_cast<long long>(h) * d.dim + i) : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const int e = threadIdx.x + u * T, tt = e >> 5, c = static_cast<int>(blockIdx.x) * 32 + (e & 31);
      rv[u] = (tt < nt && c < d.vdim) ? ld_as_float(d.v, d.in_dt, static_cast<long long>(base + t0 + tt) * d.ldv + static_cast<long long>(h) * d.vdim + c) : 0.f;
    }
    if (!PLAIN && threadIdx.x < nt) rb = ld_as_float(d.b, d.b_dt, static_cast<long long>(base + t0 + threadIdx.x) * d.ld_b + h);
  };
  fetch(0);
  for (int t0 = 0; t0 < n; t0 += CT) {
    const int nt = min(CT, n - t0);
    __syncthreads();
#pragma unroll
    for (int u = 0; u < NPF; ++u) {
      const int e = threadIdx.x + u * T, tt = e / DP, i = e - tt * DP;
      qs[tt][i] = rq[u] * q_in;
      ks[tt][i] = rk[u];
      gs[tt][i] = ra[u] == -INFINITY ? 1.f : (d.prepared ? ra[u] : expf(neg_rate * softplusf_(ra[u])));
    }
#pragma unroll
    for (int u = 0; u < NV; ++u) vs[threadIdx.x + u * T] = rv[u];
    if (!PLAIN && threadIdx.x < nt) betas[threadIdx.x] = d.prepared ? rb : sigmoidf_(rb);
    __syncthreads();
    for (int tt = (PLAIN || d.prepared) ? nt : warp; tt < nt; tt += nwarps) {
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < DP; i += 32) {
        sq = fmaf(qs[tt][i], qs[tt][i], sq);
        sk = fmaf(ks[tt][i], ks[tt][i], sk);
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float qn = qscale / sqrtf(sq + d.unit_eps), kn = 1.f / sqrtf(sk + d.unit_eps);
      for (int i = lane; i < DP; i += 32) {
        qs[tt][i] *= qn;
        ks[tt][i] *= kn;
      }
    }
    __syncthreads();
    if (t0 + CT < n) fetch(t0 + CT);
    for (int tt = 0; tt < nt; ++tt) {
      const long long row = base + t0 + tt;
      const float vj = vs[tt * 32 + col];
      float4 k4[NM];
      float r0 = 0.f, r1 = 0.f;
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        const float4 g4 = *reinterpret_cast<const float4*>(&gs[tt][4 * LANES * m + 4 * part]);
        k4[m] = *reinterpret_cast<const float4*>(&ks[tt][4 * LANES * m + 4 * part]);
        S[m][0] *= g4.x; S[m][1] *= g4.y; S[m][2] *= g4.z; S[m][3] *= g4.w;
        if constexpr (!PLAIN) {
          r0 = fmaf(S[m][0], k4[m].x, r0);
          r1 = fmaf(S[m][1], k4[m].y, r1);
          r0 = fmaf(S[m][2], k4[m].z, r0);
          r1 = fmaf(S[m][3], k4[m].w, r1);
        }
      }
      float u = vj;
      if constexpr (!PLAIN) {
        float r = r0 + r1;
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        u = betas[tt] * (vj - r);
      }
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][4 * LANES * m + 4 * part]);
        S[m][0] = fmaf(k4[m].x, u, S[m][0]);
        S[m][1] = fmaf(k4[m].y, u, S[m][1]);
        S[m][2] = fmaf(k4[m].z, u, S[m][2]);
        S[m][3] = fmaf(k4[m].w, u, S[m][3]);
        o0 = fmaf(S[m][0], q4.x, o0);
        o1 = fmaf(S[m][1], q4.y, o1);
        o0 = fmaf(S[m][2], q4.z, o0);
        o1 = fmaf(S[m][3], q4.w, o1);
      }
      float o = o0 + o1;
#pragma unroll
      for (int x = 1; x < LANES; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
      if (active && part == 0) st_from_float(d.out, d.out_dt, row * d.ld_out + static_cast<long long>(h) * d.vdim + j, o);
    }
  }
  if (active) {
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * LANES * m + 4 * part + e;
        if (i < d.dim) sp[static_cast<long long>(i) * d.vdim] = S[m][e];
      }
  }
}

// the delta rule's per-token inputs, all tokens in parallel: one warp per (token, head) writes the head's decays and write strength,
// and for the first head of each q / k group the group's unit vectors (q also times dim^-1/2)
struct DeltaPrepDev {
  long long rows;
  const void* q; long long ldq; const void* k; long long ldk; int in_dt;
  const void* a; long long ld_a; int a_dt;
  const void* b; long long ld_b; int b_dt;
  const void* a_log; int a_log_dt;
  int heads, kv_heads, dim;
  float unit_eps;
  float* qn; float* kn; float* g; float* beta;
};

__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaPrepDev d) {
  pdl_trigger();
  pdl_wait();
  const long long w = blockIdx.x * 4LL + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= d.rows * d.heads) return;
  const long long tok = w / d.heads;
  const int h = static_cast<int>(w - tok * d.heads);
  const float neg_rate = -expf(ld_as_float(d.a_log, d.a_log_dt, h));
  for (int i = lane; i < d.dim; i += 32)
    d.g[(tok * d.heads + h) * d.dim + i] = expf(neg_rate * softplusf_(ld_as_float(d.a, d.a_dt, tok * d.ld_a + static_cast<long long>(h) * d.dim + i)));
  if (lane == 0) d.beta[tok * d.heads + h] = sigmoidf_(ld_as_float(d.b, d.b_dt, tok * d.ld_b + h));
  const int rep = d.heads / d.kv_heads;
  if (h % rep) return;
  const int gq = h / rep;
  float sq = 0.f, sk = 0.f;
  for (int i = lane; i < d.dim; i += 32) {
    const float qv = ld_as_float(d.q, d.in_dt, tok * d.ldq + static_cast<long long>(gq) * d.dim + i);
    const float kv = ld_as_float(d.k, d.in_dt, tok * d.ldk + static_cast<long long>(gq) * d.dim + i);
    sq = fmaf(qv, qv, sq);
    sk = fmaf(kv, kv, sk);
  }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  const float qn = 1.f / sqrtf(static_cast<float>(d.dim)) / sqrtf(sq + d.unit_eps), kn = 1.f / sqrtf(sk + d.unit_eps);
  for (int i = lane; i < d.dim; i += 32) {
    const long long o = (tok * d.kv_heads + gq) * d.dim + i;
    d.qn[o] = ld_as_float(d.q, d.in_dt, tok * d.ldq + static_cast<long long>(gq) * d.dim + i) * qn;
    d.kn[o] = ld_as_float(d.k, d.in_dt, tok * d.ldk + static_cast<long long>(gq) * d.dim + i) * kn;
  }
}

// gated linear attention's decays, all tokens in parallel: g = sigmoid(a)^(1 / tau) = exp(-softplus(-a) / tau)
struct GlaPrepDev {
  long long rows; int width;
  const void* a; long long ld_a; int a_dt;
  float inv_tau;
  float* g;
};

__global__ void __launch_bounds__(256) gla_prep_kernel(GlaPrepDev d) {
  pdl_trigger();
  pdl_wait();
  const long long total = d.rows * d.width;
  for (long long e = blockIdx.x * 256LL + threadIdx.x; e < total; e += static_cast<long long>(gridDim.x) * 256) {
    const long long r = e / d.width;
    const int c = static_cast<int>(e - r * d.width);
    d.g[e] = expf(-softplusf_(-ld_as_float(d.a, d.a_dt, r * d.ld_a + c)) * d.inv_tau);
  }
}

static int pad_dim(int dim) { return dim <= 16 ? 16 : dim <= 32 ? 32 : dim <= 64 ? 64 : dim <= 128 ? 128 : 256; }
static int col_threads(int vdim) { return vdim <= 32 ? 32 : vdim <= 64 ? 64 : 128; }

}  // namespace vy

#define VY_NEED_DEVICE(name)                                                   \
  if (!vy_device_ok()) {                                                       \
    ::vy::set_error(name ": no sm_100 device (there is no CPU fallback)");     \
    return VY_ERR_NO_DEVICE;                                                   \
  }

extern "C" int vy_rms_norm(const VyRmsNorm* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_rms_norm: null params");
  VY_NEED_DEVICE("vy_rms_norm");
  VY_CHECK_ARG(p->tokens > 0 && p->groups > 0 && p->width > 0 && p->x && p->out, "vy_rms_norm: bad arguments");
  VY_CHECK_ARG(dtype_ok(p->x_dtype) && dtype_ok(p->out_dtype), "vy_rms_norm: bad dtype");
  VY_CHECK_ARG(p->w_mode >= 0 && p->w_mode <= 2 && (p->w_mode == 0 || (p->weight && dtype_ok(p->w_dtype))), "vy_rms_norm: bad weight");
  if (p->gate) VY_CHECK_ARG(dtype_ok(p->gate_dtype), "vy_rms_norm: bad gate dtype");
  NormDev d;
  d.rows = static_cast<long long>(p->tokens) * p->groups; d.groups = p->groups; d.width = p->width;
  d.row_index = p->row_index;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.w = p->weight; d.w_dt = p->w_dtype; d.w_mode = p->w_mode; d.w_full = p->w_full ? 1 : 0;
  d.gate = p->gate; d.ld_gate = p->ld_gate; d.gate_dt = p->gate_dtype; d.gate_act = p->gate_act;
  d.eps = p->eps; d.coef = p->coef == 0.f ? 1.f : p->coef; d.accumulate = p->accumulate;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  VY_CHECK_ARG(!p->copy || (dtype_ok(p->copy_dtype) && p->out_dtype == VY_F32), "vy_rms_norm: the second copy goes with an fp32 out");
  d.copy = p->copy; d.ld_copy = p->ld_copy; d.copy_dt = p->copy_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  const int tpr = d.width <= 256 ? 32 : d.width <= 1024 ? 128 : d.width <= 2048 ? 256 : 0;
  const long long blocks = tpr ? (d.rows + 256 / tpr - 1) / (256 / tpr) : (d.rows + 3) / 4;
  VY_CHECK_ARG(blocks <= 2147483647LL && d.rows <= 2147483647LL, "vy_rms_norm: too many rows");
  const dim3 grid(static_cast<unsigned>(blocks));
  const auto al = [](const void* q, size_t a) { return reinterpret_cast<uintptr_t>(q) % a == 0; };
  const bool vec = d.x_dt == VY_F32 && d.width % 4 == 0 && d.ldx % 4 == 0 && al(d.x, 16) &&
                   (!d.gate || (d.gate_dt == VY_F32 && d.ld_gate % 4 == 0 && al(d.gate, 16))) && d.ld_out % 4 == 0 &&
                   (d.out_dt == VY_F32 ? al(d.out, 16) : (al(d.out, 8) && !d.accumulate));
  if (tpr == 32) VY_CUDA_OK(vec ? launch_kernel(rms_norm_cached_kernel<32, true>, grid, dim3(256), 0, st, d)
                                : launch_kernel(rms_norm_cached_kernel<32, false>, grid, dim3(256), 0, st, d));
  else if (tpr == 128) VY_CUDA_OK(vec ? launch_kernel(rms_norm_cached_kernel<128, true>, grid, dim3(256), 0, st, d)
                                      : launch_kernel(rms_norm_cached_kernel<128, false>, grid, dim3(256), 0, st, d));
  else if (tpr == 256) VY_CUDA_OK(vec ? launch_kernel(rms_norm_cached_kernel<256, true>, grid, dim3(256), 0, st, d)
                                      : launch_kernel(rms_norm_cached_kernel<256, false>, grid, dim3(256), 0, st, d));
  else VY_CUDA_OK(launch_kernel(rms_norm_kernel, grid, dim3(128), 0, st, d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_kv_page_write(const VyKvWrite* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_kv_page_write: null params");
  VY_NEED_DEVICE("vy_kv_page_write");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->block_table && p->block_size > 0 &&
                   p->table_width > 0, "vy_kv_page_write: bad batch");
  VY_CHECK_ARG(p->k && p->v && p->k_pool && p->v_pool && p->k_width > 0 && p->v_width > 0 && dtype_ok(p->in_dtype) && dtype_ok(p->pool_dtype),
               "vy_kv_page_write: bad tensors");
  KvwDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.table = p->block_table; d.tw = p->table_width; d.bs = p->block_size;
  d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype;
  d.kw = p->k_width; d.vw = p->v_width;
  d.kp = p->k_pool; d.vp = p->v_pool; d.pool_dt = p->pool_dtype;
  const int gx = p->max_new < 4096 ? p->max_new : 4096;
  VY_CUDA_OK(launch_kernel(kv_page_write_kernel, dim3(gx, p->n_seqs), dim3(128), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int64_t vy_window_attn_workspace_floats(int32_t n_seqs, int32_t heads, int32_t kv_heads, int32_t vdim) {
  if (n_seqs <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || vdim <= 0) return 0;
  return vy::window_attn_heads_workspace_floats(n_seqs, heads, kv_heads, vdim);
}

extern "C" int vy_window_attn(const VyWinAttn* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_window_attn: null params");
  VY_NEED_DEVICE("vy_window_attn");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->block_table && p->block_size > 0 &&
                   p->table_width > 0, "vy_window_attn: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->kv_heads > 0 && p->heads % p->kv_heads == 0 && p->heads <= 65535 && p->dim > 0 && p->vdim > 0 &&
                   p->vdim <= 32 * WA_VR, "vy_window_attn: bad head geometry (heads %d, kv_heads %d, dim %d, vdim %d <= %d)", p->heads,
               p->kv_heads, p->dim, p->vdim, 32 * WA_VR);
  VY_CHECK_ARG(p->q && p->k_pool && p->v_pool && p->out && dtype_ok(p->q_dtype) && dtype_ok(p->pool_dtype) && dtype_ok(p->out_dtype),
               "vy_window_attn: bad tensors");
  VY_CHECK_ARG(p->keep_first >= 0, "vy_window_attn: negative keep_first");
  if (p->sink) VY_CHECK_ARG(dtype_ok(p->sink_dtype), "vy_window_attn: bad sink dtype");
  if (p->gate) VY_CHECK_ARG(dtype_ok(p->gate_dtype), "vy_window_attn: bad gate dtype");
  WinDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.table = p->block_table; d.tw = p->table_width; d.bs = p->block_size;
  d.q = p->q; d.ldq = p->ldq; d.q_dt = p->q_dtype;
  d.kp = p->k_pool; d.vp = p->v_pool; d.pool_dt = p->pool_dtype;
  d.k_row = p->k_row > 0 ? p->k_row : static_cast<long long>(p->kv_heads) * p->dim;
  d.v_row = p->v_row > 0 ? p->v_row : static_cast<long long>(p->kv_heads) * p->vdim;
  VY_CHECK_ARG(d.k_row >= static_cast<long long>(p->kv_heads) * p->dim && d.v_row >= static_cast<long long>(p->kv_heads) * p->vdim,
               "vy_window_attn: pool row strides smaller than the rows");
  d.heads = p->heads; d.kv_heads = p->kv_heads; d.dim = p->dim; d.vdim = p->vdim;
  d.scale = p->scale; d.window = p->window; d.keep = p->keep_first;
  VY_CHECK_ARG(p->chunk >= 0 && (p->chunk == 0 || (p->window <= 0 && p->keep_first == 0)), "vy_window_attn: a chunk size goes without a window and kept tokens");
  d.chunk = p->chunk;
  d.out_scale = p->out_scale == 0.f ? 1.f : p->out_scale;
  d.sink = p->sink; d.sink_dt = p->sink_dtype;
  d.gate = p->gate; d.ld_gate = p->ld_gate; d.gate_dt = p->gate_dtype;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  VY_CHECK_ARG(p->dim <= 32 * WA_VR, "vy_window_attn: dim %d > %d", p->dim, 32 * WA_VR);
  if (p->max_new >= WA_TILED_MIN) {   // prompt-sized: 64 x 64 register-tiled form
    VY_CUDA_OK(launch_window_attn_tiled(d, p->n_seqs, p->max_new, st));
  } else if (p->max_new == 1 && window_attn_heads_applies(d)) {
    int launches = 1;
    VY_CUDA_OK(launch_window_attn_heads(d, p->n_seqs, p->workspace, p->workspace_floats, st, &launches));
    VY_LAUNCH_OK();
    count_launch(launches);
    return VY_OK;
  } else if (p->max_new == 1) {
    const auto al = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    const bool vec = p->pool_dtype == VY_F32 && p->dim % 4 == 0 && p->vdim % 4 == 0 && d.k_row % 4 == 0 && d.v_row % 4 == 0 && al(p->k_pool) && al(p->v_pool);
    // four heads of one key / value head per CTA while that still leaves a CTA for most SMs; else one head per CTA
    const int per_kv = p->heads / p->kv_heads;
    const bool grouped = per_kv % 4 == 0 && static_cast<long long>(p->heads / 4) * p->n_seqs >= 96;
    const int hg = grouped ? 4 : 1;
    const size_t smem = sizeof(float) * hg * (2 * WD_WARPS + static_cast<size_t>(WD_WARPS) * p->vdim);
    const dim3 grid(1, p->heads / hg, p->n_seqs), block(WD_WARPS * 32);
    VY_CUDA_OK(grouped ? (vec ? launch_kernel(window_attn_decode_kernel<true, 4>, grid, block, smem, st, d)
                              : launch_kernel(window_attn_decode_kernel<false, 4>, grid, block, smem, st, d))
                       : (vec ? launch_kernel(window_attn_decode_kernel<true, 1>, grid, block, smem, st, d)
                              : launch_kernel(window_attn_decode_kernel<false, 1>, grid, block, smem, st, d)));
  } else {
    const size_t smem = sizeof(float) * static_cast<size_t>(WA_WARPS) * p->dim;
    VY_CUDA_OK(launch_kernel(window_attn_kernel, dim3((p->max_new + WA_WARPS - 1) / WA_WARPS, p->heads, p->n_seqs), dim3(WA_WARPS * 32), smem,
                             st, d));
  }
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_causal_conv(const VyCausalConv* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_causal_conv: null params");
  VY_NEED_DEVICE("vy_causal_conv");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->slot, "vy_causal_conv: bad batch");
  VY_CHECK_ARG(p->channels > 0 && p->taps >= 1 && p->taps <= CONV_MAX_TAPS, "vy_causal_conv: channels %d, taps %d (1..%d)", p->channels,
               p->taps, CONV_MAX_TAPS);
  VY_CHECK_ARG(p->x && p->w && p->out && p->x != p->out && (p->state || p->taps == 1) && dtype_ok(p->x_dtype) && dtype_ok(p->w_dtype) &&
                   dtype_ok(p->out_dtype), "vy_causal_conv: bad tensors");
  VY_CHECK_ARG((p->max_new + CONV_TOK - 1) / CONV_TOK <= 65535, "vy_causal_conv: too many tokens per sequence");
  ConvDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.slot = p->slot;
  d.channels = p->channels; d.taps = p->taps;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.w = p->w; d.w_dt = p->w_dtype;
  d.state = p->state; d.act = p->act;
  d.fuse_state = p->max_new <= CONV_TOK ? 1 : 0;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  const int cb = (p->channels + 127) / 128;
  VY_CUDA_OK(launch_kernel(causal_conv_kernel, dim3(cb, (p->max_new + CONV_TOK - 1) / CONV_TOK, p->n_seqs), dim3(128), 0, st, d));
  VY_LAUNCH_OK();
  count_launch();
  if (p->taps > 1 && !d.fuse_state) {
    VY_CUDA_OK(launch_kernel(causal_conv_state_kernel, dim3(cb, p->n_seqs), dim3(128), 0, st, d));
    VY_LAUNCH_OK();
    count_launch();
  }
  return VY_OK;
}

namespace vy {
template <int DP>
static cudaError_t launch_linear_attn(const RecDev& d, int n_seqs, cudaStream_t st) {
  const int threads = col_threads(d.vdim);
  return launch_kernel(linear_attn_kernel<DP>, dim3((d.vdim + threads - 1) / threads, d.heads, n_seqs), dim3(threads), 0, st, d);
}
template <int DP, bool PLAIN = false>
static cudaError_t launch_delta_rule(const RecDev& d, int n_seqs, cudaStream_t st) {
  const int threads = 32 * DeltaLanes<DP>::value;   // 32 state columns per CTA
  constexpr int CT = RecChunk<DP>::CT;
  const size_t smem = sizeof(float) * (3 * CT * DP + CT + CT * 32);
  const int cols = 32;
  if (DP >= 256) {
    static bool once = false;
    if (!once) {
      cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<DP, PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
      if (e != cudaSuccess) return e;
      once = true;
    }
  }
  return launch_kernel(delta_rule_kernel<DP, PLAIN>, dim3((d.vdim + cols - 1) / cols, d.heads, n_seqs), dim3(threads), smem, st, d);
}
}  // namespace vy

extern "C" int vy_linear_attn(const VyLinAttn* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_linear_attn: null params");
  VY_NEED_DEVICE("vy_linear_attn");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->cu_tokens && p->pos0 && p->slot, "vy_linear_attn: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->dim <= 256 && p->vdim > 0, "vy_linear_attn: heads %d, dim %d (<= 256), vdim %d",
               p->heads, p->dim, p->vdim);
  VY_CHECK_ARG(p->q && p->k && p->v && p->decay && p->state && p->out && dtype_ok(p->in_dtype) && dtype_ok(p->out_dtype),
               "vy_linear_attn: bad tensors");
  RecDev d;
  memset(&d, 0, sizeof(d));
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.slot = p->slot;
  d.q = p->q; d.ldq = p->ldq; d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype; d.in_act = p->in_act;
  d.decay = p->decay;
  d.heads = p->heads; d.kv_heads = p->heads; d.dim = p->dim; d.vdim = p->vdim;
  d.state = p->state;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  cudaError_t e;
  if (p->max_new >= LA_CHUNKED_MIN && p->dim <= 128) {
    e = launch_linear_attn_chunked(d, p->n_seqs, st);
  } else switch (pad_dim(p->dim)) {
    case 16: e = launch_linear_attn<16>(d, p->n_seqs, st); break;
    case 32: e = launch_linear_attn<32>(d, p->n_seqs, st); break;
    case 64: e = launch_linear_attn<64>(d, p->n_seqs, st); break;
    case 128: e = launch_linear_attn<128>(d, p->n_seqs, st); break;
    default: e = launch_linear_attn<256>(d, p->n_seqs, st); break;
  }
  VY_CUDA_OK(e);
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int64_t vy_delta_rule_workspace_floats(int64_t rows, int32_t heads, int32_t kv_heads, int32_t dim) {
  return rows * (2LL * kv_heads * dim + static_cast<int64_t>(heads) * dim + heads);
}

extern "C" int vy_delta_rule(const VyDeltaRule* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_delta_rule: null params");
  VY_NEED_DEVICE("vy_delta_rule");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->cu_tokens && p->pos0 && p->slot, "vy_delta_rule: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->heads <= 65535 && p->kv_heads > 0 && p->heads % p->kv_heads == 0 && p->dim > 0 && p->dim <= 256 && p->vdim > 0,
               "vy_delta_rule: heads %d, kv_heads %d, dim %d (<= 256), vdim %d", p->heads, p->kv_heads, p->dim, p->vdim);
  VY_CHECK_ARG(p->q && p->k && p->v && p->a && p->b && p->a_log && p->state && p->out && dtype_ok(p->in_dtype) && dtype_ok(p->a_dtype) &&
                   dtype_ok(p->b_dtype) && dtype_ok(p->a_log_dtype) && dtype_ok(p->out_dtype), "vy_delta_rule: bad tensors");
  RecDev d;
  memset(&d, 0, sizeof(d));
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.slot = p->slot;
  d.q = p->q; d.ldq = p->ldq; d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype;
  d.a = p->a; d.ld_a = p->ld_a; d.a_dt = p->a_dtype;
  d.b = p->b; d.ld_b = p->ld_b; d.b_dt = p->b_dtype;
  d.a_log = p->a_log; d.a_log_dt = p->a_log_dtype;
  d.heads = p->heads; d.kv_heads = p->kv_heads; d.dim = p->dim; d.vdim = p->vdim;
  d.unit_eps = p->unit_eps;
  d.state = p->state;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  if (p->workspace && p->rows > 0 && p->in_dtype == VY_F32 && p->workspace_floats >= vy_delta_rule_workspace_floats(p->rows, p->heads, p->kv_heads, p->dim)) {
    DeltaPrepDev pd;
    pd.rows = p->rows;
    pd.q = p->q; pd.ldq = p->ldq; pd.k = p->k; pd.ldk = p->ldk; pd.in_dt = p->in_dtype;
    pd.a = p->a; pd.ld_a = p->ld_a; pd.a_dt = p->a_dtype;
    pd.b = p->b; pd.ld_b = p->ld_b; pd.b_dt = p->b_dtype;
    pd.a_log = p->a_log; pd.a_log_dt = p->a_log_dtype;
    pd.heads = p->heads; pd.kv_heads = p->kv_heads; pd.dim = p->dim; pd.unit_eps = p->unit_eps;
    const long long qk = p->rows * p->kv_heads * p->dim, hg = p->rows * p->heads * p->dim;
    pd.qn = p->workspace; pd.kn = pd.qn + qk; pd.g = pd.kn + qk; pd.beta = pd.g + hg;
    const long long blocks = (p->rows * p->heads + 3) / 4;
    VY_CHECK_ARG(blocks <= 2147483647LL, "vy_delta_rule: too many rows");
    VY_CUDA_OK(launch_kernel(delta_prep_kernel, dim3(static_cast<unsigned>(blocks)), dim3(128), 0, st, pd));
    VY_LAUNCH_OK();
    count_launch();
    d.q = pd.qn; d.ldq = static_cast<long long>(p->kv_heads) * p->dim; d.k = pd.kn; d.ldk = d.ldq; 
    d.a = pd.g; d.ld_a = static_cast<long long>(p->heads) * p->dim; d.a_dt = VY_F32;
    d.b = pd.beta; d.ld_b = p->heads; d.b_dt = VY_F32;
    d.prepared = 1;
  }
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaError_t e;
  switch (pad_dim(p->dim)) {
    case 16: e = launch_delta_rule<16>(d, p->n_seqs, st); break;
    case 32: e = launch_delta_rule<32>(d, p->n_seqs, st); break;
    case 64: e = launch_delta_rule<64>(d, p->n_seqs, st); break;
    case 128: e = launch_delta_rule<128>(d, p->n_seqs, st); break;
    default: e = launch_delta_rule<256>(d, p->n_seqs, st); break;
  }
  VY_CUDA_OK(e);
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_gated_linear_attn(const VyGatedLinAttn* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_gated_linear_attn: null params");
  VY_NEED_DEVICE("vy_gated_linear_attn");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->cu_tokens && p->pos0 && p->slot, "vy_gated_linear_attn: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->dim <= 256 && p->vdim > 0 && p->tau > 0.f,
               "vy_gated_linear_attn: heads %d, dim %d (<= 256), vdim %d, tau %g (> 0)", p->heads, p->dim, p->vdim, static_cast<double>(p->tau));
  VY_CHECK_ARG(p->q && p->k && p->v && p->a && p->state && p->out && dtype_ok(p->in_dtype) && dtype_ok(p->a_dtype) && dtype_ok(p->out_dtype),
               "vy_gated_linear_attn: bad tensors");
  const long long width = static_cast<long long>(p->heads) * p->dim;
  VY_CHECK_ARG(p->rows > 0 && p->workspace && p->workspace_floats >= p->rows * width, "vy_gated_linear_attn: the workspace holds rows * heads * dim floats");
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  GlaPrepDev pd;
  pd.rows = p->rows; pd.width = static_cast<int>(width);
  pd.a = p->a; pd.ld_a = p->ld_a; pd.a_dt = p->a_dtype;
  pd.inv_tau = 1.f / p->tau;
  pd.g = p->workspace;
  const long long blocks = (p->rows * width + 255) / 256;
  VY_CUDA_OK(launch_kernel(gla_prep_kernel, dim3(static_cast<unsigned>(blocks < 65535 * 16 ? blocks : 65535 * 16)), dim3(256), 0, st, pd));
  VY_LAUNCH_OK();
  count_launch();
  RecDev d;
  memset(&d, 0, sizeof(d));
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.slot = p->slot;
  d.q = p->q; d.ldq = p->ldq; d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype;
  d.a = pd.g; d.ld_a = width; d.a_dt = VY_F32;
  d.heads = p->heads; d.kv_heads = p->heads; d.dim = p->dim; d.vdim = p->vdim;
  d.prepared = 1;
  d.q_scale = p->q_scale == 0.f ? 1.f : p->q_scale;
  d.state = p->state;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaError_t e;
  switch (pad_dim(p->dim)) {
    case 16: e = launch_delta_rule<16, true>(d, p->n_seqs, st); break;
    case 32: e = launch_delta_rule<32, true>(d, p->n_seqs, st); break;
    case 64: e = launch_delta_rule<64, true>(d, p->n_seqs, st); break;
    case 128: e = launch_delta_rule<128, true>(d, p->n_seqs, st); break;
    default: e = launch_delta_rule<256, true>(d, p->n_seqs, st); break;
  }
  VY_CUDA_OK(e);
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

// Pieces of decoder layers whose sublayers run side by side on one normed input, over a packed batch:
//   * layer norm with weight and bias (fp32 mean and mean squared deviation, two passes over a row held in shared memory);
//   * the layer's close: residual + sigmoid-gated sublayer results, stored as the layer's own result in a stack of all earlier
//     results, the coefficient-weighted sum over that stack handed on, and (fused) the NEXT layer's norm of that sum, so a layer
//     boundary is one launch and one pass over the row;
//   * the gated experts' activation (clamped gate and up halves, g sigmoid(alpha g) (u + 1)) with each token's routing weights;
//   * pair rotation of queries and keys by position fused with the page write of keys and values.
// Statistics, gates, sums and angles are fp32 whatever the I/O dtypes.
#include <math.h>
#include <stdint.h>

#include "seqmix.cuh"

namespace vy {

constexpr int PB_T = 128;

// sum over the CTA (any multiple of 32 threads up to 1024), the same value in every thread
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();   // red may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int w = 0; w < nw; ++w) s += red[w];
  return s;
}

struct MixDev {
  long long rows; int width;
  const int* row_index;
  // norm-only input (any dtype) when `mix` is off
  const void* xin; long long ld_xin; int xin_dt;
  // layer close
  const float* x; long long ldx;
  const void* y1; long long ld_y1; int y1_dt; const void* g1; long long ld_g1; int g1_dt;
  const void* y2; long long ld_y2; int y2_dt; const void* g2; long long ld_g2; int g2_dt;
  float* stack; long long stack_stride; int depth; const float* coef;
  float* mixed; long long ld_mixed;
  const void* nw; const void* nb; int nw_dt; float eps;
  void* nout; long long ld_nout; int nout_dt;
};

// one CTA per row (128 to 1024 threads, about two columns per thread: the loads of a column cannot pass the stores of the one before,
// so few columns per thread keep the row's loads in flight together); the row's fp32 values live in shared memory between the passes
template <bool MIX>
__global__ void __launch_bounds__(1024) depth_mix_norm_kernel(MixDev d) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float pb_row[];   // [width]
  __shared__ float red[32];
  const int t = threadIdx.x, PB_T = blockDim.x;
  for (long long r = blockIdx.x; r < d.rows; r += gridDim.x) {
    __syncthreads();   // the previous row's readers are done with pb_row
    if (MIX) {
      for (int c = t; c < d.width; c += PB_T) {
        float v = d.x[r * d.ldx + c];
        const float a = ld_as_float(d.y1, d.y1_dt, r * d.ld_y1 + c);
        v += d.g1 ? a * sigmoidf_(ld_as_float(d.g1, d.g1_dt, r * d.ld_g1 + c)) : a;
        if (d.y2) {
          const float b = ld_as_float(d.y2, d.y2_dt, r * d.ld_y2 + c);
          v += d.g2 ? b * sigmoidf_(ld_as_float(d.g2, d.g2_dt, r * d.ld_g2 + c)) : b;
        }
        if (d.stack) {
          const long long o = r * d.width + c;
          d.stack[static_cast<long long>(d.depth - 1) * d.stack_stride + o] = v;
          float m = 0.f;
          for (int j = 0; j < d.depth - 1; ++j) m = fmaf(d.coef[j], d.stack[j * d.stack_stride + o], m);
          v = fmaf(d.coef[d.depth - 1], v, m);
        }
        if (d.mixed) d.mixed[r * d.ld_mixed + c] = v;
        pb_row[c] = v;
      }
    } else {
      const long long src = d.row_index ? d.row_index[r] : r;
      for (int c = t; c < d.width; c += PB_T) pb_row[c] = ld_as_float(d.xin, d.xin_dt, src * d.ld_xin + c);
    }
    if (!d.nout) continue;
    float s = 0.f;
    __syncthreads();
    for (int c = t; c < d.width; c += PB_T) s += pb_row[c];
    const float mean = block_sum(s, red) / static_cast<float>(d.width);
    float q = 0.f;
    for (int c = t; c < d.width; c += PB_T) {
      const float u = pb_row[c] - mean;
      q = fmaf(u, u, q);
    }
    const float inv = 1.f / sqrtf(block_sum(q, red) / static_cast<float>(d.width) + d.eps);
    for (int c = t; c < d.width; c += PB_T) {
      float v = (pb_row[c] - mean) * inv;
      if (d.nw) v *= ld_as_float(d.nw, d.nw_dt, c);
      if (d.nb) v += ld_as_float(d.nb, d.nw_dt, c);
      st_from_float(d.nout, d.nout_dt, r * d.ld_nout + c, v);
    }
  }
}

// ---- gated experts' activation ------------------------------------------------------------------------------------------------
struct GluDev {
  long long rows; int experts, ff, shared_ff;
  const void* h; long long ldh; int h_dt;
  const float* dense; long long ld_dense;
  float limit, shared_limit, alpha;
  void* out; long long ld_out; int out_dt;
};

__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return g * sigmoidf_(alpha * g) * (u + 1.f);
}

// blockIdx.x = token, threads (and blockIdx.y) over output columns. VEC: 8 adjacent columns per thread with 16 / 32-byte accesses
// (ff and shared_ff multiples of 8, aligned rows); an unchosen expert's columns are written 0 without reading its hidden values.
template <bool VEC>
__global__ void __launch_bounds__(256) moe_glu_kernel(GluDev d) {
  pdl_trigger();
  pdl_wait();
  const long long r = blockIdx.x;
  const int ecols = d.experts * d.ff, cols = ecols + d.shared_ff;
  if (VEC) {
    for (int c0 = (blockIdx.y * 256 + threadIdx.x) * 8; c0 < cols; c0 += gridDim.y * 256 * 8) {
      float y[8];
      const bool routed = c0 < ecols;
      const int e = routed ? c0 / d.ff : d.experts;
      const int j = routed ? c0 - e * d.ff : c0 - ecols;
      const int half = routed ? d.ff : d.shared_ff;
      const float w = routed ? (d.dense ? d.dense[r * d.ld_dense + e] : 1.f) : 1.f;
      if (w != 0.f) {
        const long long o = r * d.ldh + static_cast<long long>(e) * 2 * d.ff + j;   // the shared block follows the experts' 2 ff columns each
        float g[8], u[8];
        ld8_as_float(d.h, d.h_dt, o, g);
        ld8_as_float(d.h, d.h_dt, o + half, u);
        const float lim = routed ? d.limit : d.shared_limit;
#pragma unroll
        for (int k = 0; k < 8; ++k) y[k] = w * clamped_glu(g[k], u[k], lim, d.alpha);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) y[k] = 0.f;
      }
      st8_from_float(d.out, d.out_dt, r * d.ld_out + c0, y);
    }
    return;
  }
  for (int c = blockIdx.y * 256 + threadIdx.x; c < cols; c += gridDim.y * 256) {
    float y = 0.f;
    if (c < ecols) {
      const int e = c / d.ff, j = c - e * d.ff;
      const float w = d.dense ? d.dense[r * d.ld_dense + e] : 1.f;
      if (w != 0.f) {
        const long long o = r * d.ldh + static_cast<long long>(e) * 2 * d.ff + j;
        y = w * clamped_glu(ld_as_float(d.h, d.h_dt, o), ld_as_float(d.h, d.h_dt, o + d.ff), d.limit, d.alpha);
      }
    } else {
      const int j = c - ecols;
      const long long o = r * d.ldh + static_cast<long long>(d.experts) * 2 * d.ff + j;
      y = clamped_glu(ld_as_float(d.h, d.h_dt, o), ld_as_float(d.h, d.h_dt, o + d.shared_ff), d.shared_limit, d.alpha);
    }
    st_from_float(d.out, d.out_dt, r * d.ld_out + c, y);
  }
}

// ---- rotation + page write ----------------------------------------------------------------------------------------------------
struct RopeKvDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  void* q; long long ldq; const void* k; long long ldk; const void* v; long long ldv; int in_dt;
  int heads, kv_heads, dim, vdim, rot_dims;
  const float* inv_freq;
  void* kp; void* vp; int pool_dt;
};

__device__ __forceinline__ void turn_pair(float& u, float& v, int pos, float f) {
  float sn, cs;
  sincosf(static_cast<float>(pos) * f, &sn, &cs);
  const float a = u * cs - v * sn, b = v * cs + u * sn;
  u = a;
  v = b;
}

// one CTA per token: threads over the rotated pairs of q (in place), the pairs / passing entries of k and the entries of v
__global__ void __launch_bounds__(PB_T) rope_kv_write_kernel(RopeKvDev d) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  const int half = d.rot_dims / 2;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int pos = d.pos0[s] + i;
    const long long prow = static_cast<long long>(d.table[static_cast<long long>(s) * d.tw + pos / d.bs]) * d.bs + pos % d.bs;
    const long long qo = static_cast<long long>(base + i) * d.ldq, ko = static_cast<long long>(base + i) * d.ldk, vo = static_cast<long long>(base + i) * d.ldv;
    const long long kpo = prow * d.kv_heads * d.dim, vpo = prow * d.kv_heads * d.vdim;
    for (int e = threadIdx.x; e < d.heads * half; e += PB_T) {
      const int h = e / half, pr = e - h * half;
      const long long o = qo + static_cast<long long>(h) * d.dim + 2 * pr;
      float u = ld_as_float(d.q, d.in_dt, o), w = ld_as_float(d.q, d.in_dt, o + 1);
      turn_pair(u, w, pos, d.inv_freq[pr]);
      st_from_float(d.q, d.in_dt, o, u);
      st_from_float(d.q, d.in_dt, o + 1, w);
    }
    for (int e = threadIdx.x; e < d.kv_heads * half; e += PB_T) {
      const int g = e / half, pr = e - g * half;
      const int c = g * d.dim + 2 * pr;
      float u = ld_as_float(d.k, d.in_dt, ko + c), w = ld_as_float(d.k, d.in_dt, ko + c + 1);
      turn_pair(u, w, pos, d.inv_freq[pr]);
      st_from_float(d.kp, d.pool_dt, kpo + c, u);
      st_from_float(d.kp, d.pool_dt, kpo + c + 1, w);
    }
    const int rest = d.dim - d.rot_dims;
    for (int e = threadIdx.x; e < d.kv_heads * rest; e += PB_T) {
      const int g = e / rest, c = g * d.dim + d.rot_dims + (e - g * rest);
      st_from_float(d.kp, d.pool_dt, kpo + c, ld_as_float(d.k, d.in_dt, ko + c));
    }
    for (int c = threadIdx.x; c < d.kv_heads * d.vdim; c += PB_T) st_from_float(d.vp, d.pool_dt, vpo + c, ld_as_float(d.v, d.in_dt, vo + c));
  }
}

// The general form: one warp per (token, head of q or k). Pair layout (adjacent entries, or entry i with entry i + rot_dims / 2), a
// common factor on cos and sin, an RMS division of the rotated head, a final scale; keys go to their page rows (values copied beside
// them) or, without pools, to a packed tensor. A lane holds pairs lane, lane + 32, .. and passing entries rot_dims + lane, ..: dim <= 256.
struct RopeHeadsDev {
  RopeKvDev b;
  int half_layout, unit_rms;
  float eps, rot_scale, q_scale, k_scale;
  void* k_out; long long ld_k_out;
};

__global__ void __launch_bounds__(256, 4) rope_heads_kernel(RopeHeadsDev d) {
  pdl_trigger();
  pdl_wait();
  const RopeKvDev& b = d.b;
  const int s = blockIdx.y;
  const int base = b.cu[s], n = b.cu[s + 1] - base;
  const int half = b.rot_dims / 2, rest = b.dim - b.rot_dims;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int pos = b.pos0[s] + i;
    const long long row = base + i;
    long long prow = 0;
    if (b.kp) prow = static_cast<long long>(b.table[static_cast<long long>(s) * b.tw + pos / b.bs]) * b.bs + pos % b.bs;
    for (int unit = warp; unit < b.heads + b.kv_heads; unit += nwarps) {
      const bool is_q = unit < b.heads;
      const int h = is_q ? unit : unit - b.heads;
      const void* src = is_q ? b.q : b.k;
      const long long so = row * (is_q ? b.ldq : b.ldk) + static_cast<long long>(h) * b.dim;
      float pu[4], pv[4], ps[8];
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int pr = lane + 32 * r;
        pu[r] = pv[r] = 0.f;
        if (pr < half) {
          const int iu = d.half_layout ? pr : 2 * pr, iv = d.half_layout ? pr + half : 2 * pr + 1;
          const float u = ld_as_float(src, b.in_dt, so + iu), w = ld_as_float(src, b.in_dt, so + iv);
          float sn, cs;
          sincosf(static_cast<float>(pos) * b.inv_freq[pr], &sn, &cs);
          sn *= d.rot_scale;
          cs *= d.rot_scale;
          pu[r] = u * cs - w * sn;
          pv[r] = w * cs + u * sn;
          ss = fmaf(pu[r], pu[r], ss);
          ss = fmaf(pv[r], pv[r], ss);
        }
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int c = lane + 32 * r;
        ps[r] = c < rest ? ld_as_float(src, b.in_dt, so + b.rot_dims + c) : 0.f;
        ss = fmaf(ps[r], ps[r], ss);
      }
      float f = is_q ? d.q_scale : d.k_scale;
      if (d.unit_rms) f /= sqrtf(warp_sum(ss) / static_cast<float>(b.dim) + d.eps);
      void* dst;
      long long dof;
      int dt;
      if (is_q) { dst = b.q; dof = so; dt = b.in_dt; }
      else if (b.kp) { dst = b.kp; dof = (prow * b.kv_heads + h) * b.dim; dt = b.pool_dt; }
      else { dst = d.k_out; dof = row * d.ld_k_out + static_cast<long long>(h) * b.dim; dt = b.in_dt; }
      __syncwarp();   // in place: every lane has read its entries before any lane writes (pairs are private to a lane, but keep the order explicit)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int pr = lane + 32 * r;
        if (pr < half) {
          const int iu = d.half_layout ? pr : 2 * pr, iv = d.half_layout ? pr + half : 2 * pr + 1;
          st_from_float(dst, dt, dof + iu, pu[r] * f);
          st_from_float(dst, dt, dof + iv, pv[r] * f);
        }
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int c = lane + 32 * r;
        if (c < rest) st_from_float(dst, dt, dof + b.rot_dims + c, ps[r] * f);
      }
    }
    if (b.vp) {
      const long long vo = row * b.ldv, vpo = prow * b.kv_heads * b.vdim;
      for (int c = threadIdx.x; c < b.kv_heads * b.vdim; c += blockDim.x) st_from_float(b.vp, b.pool_dt, vpo + c, ld_as_float(b.v, b.in_dt, vo + c));
    }
  }
}

}  // namespace vy

#define VY_NEED_DEVICE(name)                                                   \
  if (!vy_device_ok()) {                                                       \
    ::vy::set_error(name ": no sm_100 device (there is no CPU fallback)");     \
    return VY_ERR_NO_DEVICE;                                                   \
  }

static unsigned mix_threads(int width) {
  unsigned n = 128;
  while (n < 1024 && static_cast<int>(2 * n) < width) n *= 2;
  return n;
}

static cudaError_t mix_smem_ok(size_t smem, bool mix) {
  static size_t allowed[2] = {48 * 1024, 48 * 1024};
  if (smem <= allowed[mix]) return cudaSuccess;
  cudaError_t e = mix ? cudaFuncSetAttribute(vy::depth_mix_norm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))
                      : cudaFuncSetAttribute(vy::depth_mix_norm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e == cudaSuccess) allowed[mix] = smem;
  return e;
}

extern "C" int vy_layer_norm(const VyLayerNorm* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_layer_norm: null params");
  VY_NEED_DEVICE("vy_layer_norm");
  VY_CHECK_ARG(p->tokens > 0 && p->width > 0 && p->width <= 57 * 1024, "vy_layer_norm: tokens %lld, width %d", static_cast<long long>(p->tokens), p->width);
  VY_CHECK_ARG(p->x && p->out && dtype_ok(p->x_dtype) && dtype_ok(p->out_dtype) && ((!p->weight && !p->bias) || dtype_ok(p->w_dtype)),
               "vy_layer_norm: bad tensors");
  MixDev d;
  memset(&d, 0, sizeof(d));
  d.rows = p->tokens; d.width = p->width; d.row_index = p->row_index;
  d.xin = p->x; d.ld_xin = p->ldx; d.xin_dt = p->x_dtype;
  d.nw = p->weight; d.nb = p->bias; d.nw_dt = p->w_dtype; d.eps = p->eps;
  d.nout = p->out; d.ld_nout = p->ld_out; d.nout_dt = p->out_dtype;
  const size_t smem = sizeof(float) * p->width;
  VY_CUDA_OK(mix_smem_ok(smem, false));
  const unsigned blocks = static_cast<unsigned>(p->tokens < 1048576 ? p->tokens : 1048576);
  VY_CUDA_OK(launch_kernel(depth_mix_norm_kernel<false>, dim3(blocks), dim3(mix_threads(p->width)), smem, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_depth_mix(const VyDepthMix* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_depth_mix: null params");
  VY_NEED_DEVICE("vy_depth_mix");
  VY_CHECK_ARG(p->rows > 0 && p->width > 0 && p->width <= 57 * 1024, "vy_depth_mix: rows %lld, width %d", static_cast<long long>(p->rows), p->width);
  VY_CHECK_ARG(p->x && p->y1 && dtype_ok(p->y1_dtype) && (!p->g1 || dtype_ok(p->g1_dtype)) && (!p->y2 || dtype_ok(p->y2_dtype)) &&
                   (!p->g2 || (p->y2 && dtype_ok(p->g2_dtype))), "vy_depth_mix: bad sublayer tensors");
  VY_CHECK_ARG(!p->stack || (p->depth >= 1 && p->coef && p->stack_stride >= p->rows * p->width), "vy_depth_mix: stack needs depth >= 1, coefficients and a slice stride >= rows * width");
  VY_CHECK_ARG(p->mixed || p->norm_out, "vy_depth_mix: nothing to write");
  VY_CHECK_ARG(!p->norm_out || (dtype_ok(p->norm_out_dtype) && ((!p->norm_weight && !p->norm_bias) || dtype_ok(p->norm_w_dtype))), "vy_depth_mix: bad norm tensors");
  MixDev d;
  memset(&d, 0, sizeof(d));
  d.rows = p->rows; d.width = p->width;
  d.x = p->x; d.ldx = p->ldx;
  d.y1 = p->y1; d.ld_y1 = p->ld_y1; d.y1_dt = p->y1_dtype; d.g1 = p->g1; d.ld_g1 = p->ld_g1; d.g1_dt = p->g1_dtype;
  d.y2 = p->y2; d.ld_y2 = p->ld_y2; d.y2_dt = p->y2_dtype; d.g2 = p->g2; d.ld_g2 = p->ld_g2; d.g2_dt = p->g2_dtype;
  d.stack = p->stack; d.stack_stride = p->stack_stride; d.depth = p->depth; d.coef = p->coef;
  d.mixed = p->mixed; d.ld_mixed = p->ld_mixed;
  d.nw = p->norm_weight; d.nb = p->norm_bias; d.nw_dt = p->norm_w_dtype; d.eps = p->eps;
  d.nout = p->norm_out; d.ld_nout = p->ld_norm_out; d.nout_dt = p->norm_out_dtype;
  const size_t smem = sizeof(float) * p->width;
  VY_CUDA_OK(mix_smem_ok(smem, true));
  const unsigned blocks = static_cast<unsigned>(p->rows < 1048576 ? p->rows : 1048576);
  VY_CUDA_OK(launch_kernel(depth_mix_norm_kernel<true>, dim3(blocks), dim3(mix_threads(p->width)), smem, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_moe_glu(const VyMoeGlu* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_moe_glu: null params");
  VY_NEED_DEVICE("vy_moe_glu");
  VY_CHECK_ARG(p->rows > 0 && p->rows <= 2147483647LL && p->experts >= 0 && p->shared_ff >= 0 && (p->experts == 0 || p->ff > 0) &&
                   p->experts * static_cast<long long>(p->ff) + p->shared_ff > 0, "vy_moe_glu: bad shape");
  VY_CHECK_ARG(p->h && p->out && dtype_ok(p->h_dtype) && dtype_ok(p->out_dtype), "vy_moe_glu: bad tensors");
  GluDev d;
  d.rows = p->rows; d.experts = p->experts; d.ff = p->experts ? p->ff : 1; d.shared_ff = p->shared_ff;
  d.h = p->h; d.ldh = p->ldh; d.h_dt = p->h_dtype;
  d.dense = p->dense; d.ld_dense = p->ld_dense;
  d.limit = p->limit; d.shared_limit = p->shared_limit; d.alpha = p->alpha;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  const int cols = d.experts * d.ff + d.shared_ff;
  const auto al = [](const void* q, size_t n) { return reinterpret_cast<uintptr_t>(q) % n == 0; };
  const size_t hb = p->h_dtype == VY_F32 ? 32 : 16, ob = p->out_dtype == VY_F32 ? 32 : 16;
  const bool vec = (d.experts == 0 || d.ff % 8 == 0) && d.shared_ff % 8 == 0 && p->ldh % 8 == 0 && p->ld_out % 8 == 0 && al(p->h, hb) && al(p->out, ob);
  const int per_cta = vec ? 2048 : 256;
  int gy = (cols + per_cta - 1) / per_cta;
  if (gy > 64) gy = 64;
  const dim3 grid(static_cast<unsigned>(p->rows), gy);
  VY_CUDA_OK(vec ? launch_kernel(moe_glu_kernel<true>, grid, dim3(256), 0, static_cast<cudaStream_t>(p->stream), d)
                 : launch_kernel(moe_glu_kernel<false>, grid, dim3(256), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_rope_kv_write(const VyRopeKvWrite* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_rope_kv_write: null params");
  VY_NEED_DEVICE("vy_rope_kv_write");
  const bool paged = p->k_pool != nullptr;
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0, "vy_rope_kv_write: bad batch");
  VY_CHECK_ARG(!paged || (p->block_table && p->block_size > 0 && p->table_width > 0), "vy_rope_kv_write: pools need a block table");
  VY_CHECK_ARG(p->heads >= 0 && p->kv_heads >= 0 && p->heads + p->kv_heads > 0 && p->dim > 0 && p->rot_dims >= 0 && p->rot_dims <= p->dim && p->rot_dims % 2 == 0 &&
                   (p->rot_dims == 0 || p->inv_freq), "vy_rope_kv_write: heads %d / %d, dim %d, vdim %d, rotated %d (even, <= dim)", p->heads,
               p->kv_heads, p->dim, p->vdim, p->rot_dims);
  VY_CHECK_ARG((p->heads == 0 || p->q) && (p->kv_heads == 0 || p->k) && dtype_ok(p->in_dtype), "vy_rope_kv_write: bad tensors");
  if (paged) VY_CHECK_ARG(p->v && p->v_pool && p->vdim > 0 && dtype_ok(p->pool_dtype), "vy_rope_kv_write: bad pools");
  else VY_CHECK_ARG(p->kv_heads == 0 || p->k_out, "vy_rope_kv_write: without pools the rotated keys need k_out");
  RopeKvDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.table = p->block_table; d.tw = p->table_width; d.bs = p->block_size;
  d.q = p->q; d.ldq = p->ldq; d.k = p->k; d.ldk = p->ldk; d.v = p->v; d.ldv = p->ldv; d.in_dt = p->in_dtype;
  d.heads = p->heads; d.kv_heads = p->kv_heads; d.dim = p->dim; d.vdim = p->vdim; d.rot_dims = p->rot_dims;
  d.inv_freq = p->inv_freq;
  d.kp = p->k_pool; d.vp = paged ? p->v_pool : nullptr; d.pool_dt = p->pool_dtype;
  const unsigned gx = static_cast<unsigned>(p->max_new < 65535 ? p->max_new : 65535);
  const bool general = !paged || p->half_layout || p->unit_rms || (p->rot_scale != 0.f && p->rot_scale != 1.f) || (p->q_scale != 0.f && p->q_scale != 1.f) ||
                       (p->k_scale != 0.f && p->k_scale != 1.f);
  if (general) {
    VY_CHECK_ARG(p->dim <= 256, "vy_rope_kv_write: dim %d > 256", p->dim);
    RopeHeadsDev g;
    g.b = d;
    g.half_layout = p->half_layout ? 1 : 0; g.unit_rms = p->unit_rms ? 1 : 0;
    g.eps = p->eps;
    g.rot_scale = p->rot_scale == 0.f ? 1.f : p->rot_scale;
    g.q_scale = p->q_scale == 0.f ? 1.f : p->q_scale;
    g.k_scale = p->k_scale == 0.f ? 1.f : p->k_scale;
    g.k_out = p->k_out; g.ld_k_out = p->ld_k_out;
    // single tokens: a warp per head in flight (up to 8), few CTAs; prompts: 4 warps per token, more CTAs per SM (measured: 8 warps cost
    // prompts 0.23 -> 0.34 ms over 4 launches of 8192 tokens and saved single-token steps 29 -> 21 us)
    const int units = p->heads + p->kv_heads;
    const unsigned threads = p->max_new > 1 ? 128u : 32u * static_cast<unsigned>(units < 4 ? 4 : units > 8 ? 8 : units);
    VY_CUDA_OK(launch_kernel(rope_heads_kernel, dim3(gx, p->n_seqs), dim3(threads), 0, static_cast<cudaStream_t>(p->stream), g));
  } else {
    VY_CHECK_ARG(p->heads > 0 && p->kv_heads > 0, "vy_rope_kv_write: heads");
    VY_CUDA_OK(launch_kernel(rope_kv_write_kernel, dim3(gx, p->n_seqs), dim3(PB_T), 0, static_cast<cudaStream_t>(p->stream), d));
  }
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

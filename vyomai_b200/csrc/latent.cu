// Latent attention and mixture-of-experts pieces over a packed batch: the latent page write (RMS norm of the low-rank
// latent + pair rotation of the shared key part + store at the token's page row, one launch), the query split (unrotated
// parts copied for the per-head up-projection, rotated parts rotated in place of the attention query), the sigmoid top-k
// router, the all-experts weighting used for single tokens, and the sort / gather / combine kernels used for prompts.
// Norms, angles, router scores and weights are fp32 whatever the I/O dtypes.
#include <math.h>

#include "seqmix.cuh"

namespace vy {

// (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = pos * f, cos and sin times m, all fp32
__device__ __forceinline__ void rotate_pair(float& u, float& v, int pos, float f, float m) {
  float sn, cs;
  sincosf(static_cast<float>(pos) * f, &sn, &cs);
  sn *= m;
  cs *= m;
  const float a = u * cs - v * sn, b = v * cs + u * sn;
  u = a;
  v = b;
}

// ---- latent page write ----------------------------------------------------------------------------------------------------
struct LatDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  const void* x; long long ldx; int x_dt;
  int rank, rot_dim, rot_dims;
  const float* inv_freq; float rot_scale;
  const void* w; int w_dt;
  float eps;
  void* pool; long long pool_row; int pool_dt;
  void* copy; long long ld_copy; int copy_dt;
};

__device__ __forceinline__ void lat_store(const LatDev& d, long long po, long long co, int c, float v) {
  st_from_float(d.pool, d.pool_dt, po + c, v);
  if (d.copy) st_from_float(d.copy, d.copy_dt, co + c, v);
}

// one warp per token
__global__ void __launch_bounds__(128) latent_kv_write_kernel(LatDev d) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  for (int i = blockIdx.x * 4 + warp; i < n; i += gridDim.x * 4) {
    const int pos = d.pos0[s] + i;
    const long long row = static_cast<long long>(d.table[static_cast<long long>(s) * d.tw + pos / d.bs]) * d.bs + pos % d.bs;
    const long long xo = static_cast<long long>(base + i) * d.ldx, po = row * d.pool_row, co = static_cast<long long>(base + i) * d.ld_copy;
    float ss = 0.f;
    for (int c = lane; c < d.rank; c += 32) {
      const float v = ld_as_float(d.x, d.x_dt, xo + c);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(d.rank) + d.eps);
    for (int c = lane; c < d.rank; c += 32)
      lat_store(d, po, co, c, ld_as_float(d.x, d.x_dt, xo + c) * inv * ld_as_float(d.w, d.w_dt, c));
    for (int pr = lane; 2 * pr < d.rot_dim; pr += 32) {
      float u = ld_as_float(d.x, d.x_dt, xo + d.rank + 2 * pr);
      const bool has_v = 2 * pr + 1 < d.rot_dim;
      float v = has_v ? ld_as_float(d.x, d.x_dt, xo + d.rank + 2 * pr + 1) : 0.f;
      if (2 * pr + 1 < d.rot_dims) rotate_pair(u, v, pos, d.inv_freq[pr], d.rot_scale);
      lat_store(d, po, co, d.rank + 2 * pr, u);
      if (has_v) lat_store(d, po, co, d.rank + 2 * pr + 1, v);
    }
  }
}

// ---- query split ------------------------------------------------------------------------------------------------------------
struct SplitDev {
  const int* cu; const int* pos0;
  const void* x; long long ldx; int x_dt;
  int heads, pass, rot_dim, rot_dims;
  const float* inv_freq; float rot_scale;
  void* pass_out; long long ld_pass; int pass_dt;
  void* rot_out; long long ld_rot; int rot_head, rot_col, rot_dt;
};

// one CTA per token, threads over (head, pair-or-element)
__global__ void __launch_bounds__(128) rope_split_kernel(SplitDev d) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  const int hd = d.pass + d.rot_dim;
  const int pairs = (d.rot_dim + 1) / 2;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int pos = d.pos0[s] + i;
    const long long xo = static_cast<long long>(base + i) * d.ldx;
    if (d.pass_out) {
      for (int e = threadIdx.x; e < d.heads * d.pass; e += blockDim.x) {
        const int h = e / d.pass, c = e - h * d.pass;
        st_from_float(d.pass_out, d.pass_dt, static_cast<long long>(base + i) * d.ld_pass + e,
                      ld_as_float(d.x, d.x_dt, xo + static_cast<long long>(h) * hd + c));
      }
    }
    for (int e = threadIdx.x; e < d.heads * pairs; e += blockDim.x) {
      const int h = e / pairs, pr = e - h * pairs;
      const long long src = xo + static_cast<long long>(h) * hd + d.pass + 2 * pr;
      const long long dst = static_cast<long long>(base + i) * d.ld_rot + static_cast<long long>(h) * d.rot_head + d.rot_col + 2 * pr;
      float u = ld_as_float(d.x, d.x_dt, src);
      const bool has_v = 2 * pr + 1 < d.rot_dim;
      float v = has_v ? ld_as_float(d.x, d.x_dt, src + 1) : 0.f;
      if (2 * pr + 1 < d.rot_dims) rotate_pair(u, v, pos, d.inv_freq[pr], d.rot_scale);
      st_from_float(d.rot_out, d.rot_dt, dst, u);
      if (has_v) st_from_float(d.rot_out, d.rot_dt, dst + 1, v);
    }
  }
}

// ---- router -------------------------------------------------------------------------------------------------------------------
struct RouteDev {
  long long rows; int experts, top;
  const float* logits; long long ld;
  float scale;
  int* idx; float* weight; float* dense;
  int kind, groups, keep_groups, raw;
};

constexpr int ROUTE_WARPS = 4;

// (value, index) maximum over a warp, ties to the lowest index
__device__ __forceinline__ void warp_argmax(float& bv, int& bi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
}

// one warp per row: scores in shared memory (sigmoid, or softmax over all experts), members of the groups that were not kept
// struck out, then `top` rounds of (max value, lowest index)
__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_route_kernel(RouteDev d) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float route_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long r = static_cast<long long>(blockIdx.x) * ROUTE_WARPS + warp;
  if (r >= d.rows) return;
  float* sc = route_smem + warp * (d.experts + d.groups);
  float zmax = -INFINITY, zsum = 0.f;
  if (d.kind == VY_ROUTE_SOFTMAX) {
    for (int e = lane; e < d.experts; e += 32) zmax = fmaxf(zmax, d.logits[r * d.ld + e]);
    zmax = warp_max(zmax);
    for (int e = lane; e < d.experts; e += 32) zsum += expf(d.logits[r * d.ld + e] - zmax);
    zsum = warp_sum(zsum);
  }
  for (int e = lane; e < d.experts; e += 32) {
    const float z = d.logits[r * d.ld + e];
    sc[e] = d.kind == VY_ROUTE_SOFTMAX ? expf(z - zmax) / zsum : sigmoidf_(z);
    if (d.dense) d.dense[r * d.experts + e] = 0.f;
  }
  __syncwarp();
  if (d.groups > 1) {
    float* gs = sc + d.experts;   // a group's score: its best member; -inf once the group is kept
    const int per = d.experts / d.groups;
    for (int g = lane; g < d.groups; g += 32) {
      float b = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, sc[e]);
      gs[g] = b;
    }
    __syncwarp();
    for (int k = 0; k < d.keep_groups; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < d.groups; g += 32) {
        const float v = gs[g];
        if (v > bv || (v == bv && v != -INFINITY && g < bi)) { bv = v; bi = g; }
      }
      warp_argmax(bv, bi);
      if (lane == 0 && bi < d.groups) gs[bi] = -INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < d.experts; e += 32)
      if (gs[e / per] != -INFINITY) sc[e] = -INFINITY;   // scores are positive, so a kept group never reads -inf here by itself
    __syncwarp();
  }
  float sum = 0.f;
  float my_val = 0.f;   // lane k keeps the k-th choice (top <= 32 per pass; larger tops loop)
  int my_idx = 0;
  for (int k = 0; k < d.top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < d.experts; e += 32) {
      const float v = sc[e];
      if (v > bv) { bv = v; bi = e; }   // ascending e: the lowest index of equal values stays
    }
    warp_argmax(bv, bi);
    sum += bv;
    if (lane == (k & 31)) { my_val = bv; my_idx = bi; }
    if (lane == 0) sc[bi] = -INFINITY;
    __syncwarp();
    if ((k & 31) == 31 || k == d.top - 1) {
      // flush this group of up to 32 choices once the sum is final: groups before the last are normalised below
      const int k0 = k & ~31;
      if (k0 + lane <= k) {
        d.idx[r * d.top + k0 + lane] = my_idx;
        d.weight[r * d.top + k0 + lane] = my_val;   // raw score for now
      }
    }
  }
  __syncwarp();
  const float norm = d.raw ? d.scale : d.scale / (sum + 1e-20f);
  for (int k = lane; k < d.top; k += 32) {
    const float w = d.weight[r * d.top + k] * norm;
    d.weight[r * d.top + k] = w;
    if (d.dense) d.dense[r * d.experts + d.idx[r * d.top + k]] = w;
  }
}

// ---- all-experts weighting ----------------------------------------------------------------------------------------------------
struct ScaleDev {
  long long rows; int experts, ff, shared_ff;
  const void* h; long long ldh; int h_dt;
  const float* dense;
  const float* sg; long long ld_sg;
  void* out; long long ld_out; int out_dt;
};

// one CTA row per token (blockIdx.x), 8 consecutive columns per thread; VEC: 16-byte (bf16) / 32-byte (fp32) accesses
template <bool VEC>
__global__ void __launch_bounds__(256) moe_scale_kernel(ScaleDev d) {
  pdl_trigger();
  pdl_wait();
  const int cols = d.experts * d.ff + d.shared_ff, ecols = d.experts * d.ff;
  const long long r = blockIdx.x;
  const float sgw = d.sg ? sigmoidf_(d.sg[r * d.ld_sg]) : 1.f;
  const float* dw = d.dense + r * d.experts;
  for (int c0 = (blockIdx.y * 256 + threadIdx.x) * 8; c0 < cols; c0 += gridDim.y * 256 * 8) {
    float w[8];
    bool any = false;
    if (VEC && d.ff % 8 == 0 && ecols % 8 == 0) {   // the 8 columns belong to one expert (or all to the shared one)
      const float w0 = c0 < ecols ? dw[c0 / d.ff] : sgw;
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = w0;
      any = w0 != 0.f;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = c0 + j;
        w[j] = c < ecols ? dw[c / d.ff] : sgw;
        any |= c < cols && w[j] != 0.f;
      }
    }
    float v[8];
    if (VEC) {
      if (any) ld8_as_float(d.h, d.h_dt, r * d.ldh + c0, v);   // an unchosen expert's columns are written 0 without being read
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = w[j] == 0.f ? 0.f : v[j] * w[j];
      st8_from_float(d.out, d.out_dt, r * d.ld_out + c0, v);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c0 + j < cols)
          st_from_float(d.out, d.out_dt, r * d.ld_out + c0 + j, w[j] == 0.f ? 0.f : ld_as_float(d.h, d.h_dt, r * d.ldh + c0 + j) * w[j]);
    }
  }
}

// ---- sorted form ----------------------------------------------------------------------------------------------------------------
struct SortDev {
  long long pairs; int experts, top;
  const int* idx;
  int* counts; int* offsets; int* perm; int* inv;
};

// One CTA: count, scan, then a stable placement (each thread owns a contiguous run of pairs, so pairs of an expert keep
// their order). Prompt-sized steps hold at most a few hundred thousand pairs; the kernel is a small fraction of the experts' work.
constexpr int SORT_T = 1024;
__global__ void __launch_bounds__(SORT_T) moe_sort_kernel(SortDev d) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ int sort_smem[];   // [experts] running offsets
  const int t = threadIdx.x;
  for (int e = t; e < d.experts; e += SORT_T) d.counts[e] = 0;
  __syncthreads();
  for (long long i = t; i < d.pairs; i += SORT_T) atomicAdd(&d.counts[d.idx[i]], 1);
  __syncthreads();
  if (t == 0) {
    int at = 0;
    for (int e = 0; e < d.experts; ++e) {
      d.offsets[e] = at;
      sort_smem[e] = at;
      at += d.counts[e];
    }
    d.offsets[d.experts] = at;
  }
  __syncthreads();
  // stable placement: expert by expert would be O(experts * pairs); instead each warp takes one expert at a time and walks
  // the pairs in order with a ballot prefix
  const int warp = t >> 5, lane = t & 31;
  for (int e = warp; e < d.experts; e += SORT_T / 32) {
    int at = sort_smem[e];
    for (long long i0 = 0; i0 < d.pairs; i0 += 32) {
      const long long i = i0 + lane;
      const bool mine = i < d.pairs && d.idx[i] == e;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int dst = at + __popc(m & ((1u << lane) - 1u));
        d.perm[dst] = static_cast<int>(i);
        d.inv[i] = dst;
      }
      at += __popc(m);
    }
  }
}

struct GatherDev {
  long long n; int top, width;
  const int* perm;
  const void* x; long long ldx; int x_dt;
  void* out; long long ld_out; int out_dt;
};

__global__ void __launch_bounds__(128) moe_gather_kernel(GatherDev d) {
  pdl_trigger();
  pdl_wait();
  for (long long i = blockIdx.x; i < d.n; i += gridDim.x) {
    const long long src = d.perm[i] / d.top;
    for (int c = threadIdx.x; c < d.width; c += blockDim.x)
      st_from_float(d.out, d.out_dt, i * d.ld_out + c, ld_as_float(d.x, d.x_dt, src * d.ldx + c));
  }
}

struct CombineDev {
  long long rows; int top, width;
  const int* inv; const float* weight;
  const void* part; long long ld_part; int part_dt;
  const void* addend; long long ld_addend; int addend_dt;
  void* out; long long ld_out; int out_dt;
};

__global__ void __launch_bounds__(128) moe_combine_kernel(CombineDev d) {
  pdl_trigger();
  pdl_wait();
  for (long long r = blockIdx.x; r < d.rows; r += gridDim.x) {
    for (int c = threadIdx.x; c < d.width; c += blockDim.x) {
      float acc = d.addend ? ld_as_float(d.addend, d.addend_dt, r * d.ld_addend + c) : 0.f;
      for (int k = 0; k < d.top; ++k)
        acc = fmaf(d.weight[r * d.top + k], ld_as_float(d.part, d.part_dt, static_cast<long long>(d.inv[r * d.top + k]) * d.ld_part + c), acc);
      st_from_float(d.out, d.out_dt, r * d.ld_out + c, acc);
    }
  }
}

}  // namespace vy

#define VY_NEED_DEVICE(name)                                                   \
  if (!vy_device_ok()) {                                                       \
    ::vy::set_error(name ": no sm_100 device (there is no CPU fallback)");     \
    return VY_ERR_NO_DEVICE;                                                   \
  }

extern "C" int vy_latent_kv_write(const VyLatentWrite* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_latent_kv_write: null params");
  VY_NEED_DEVICE("vy_latent_kv_write");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->block_table && p->block_size > 0 &&
                   p->table_width > 0, "vy_latent_kv_write: bad batch");
  VY_CHECK_ARG(p->rank > 0 && p->rot_dim >= 0 && p->rot_dims >= 0 && p->rot_dims <= p->rot_dim && p->rot_dims % 2 == 0 &&
                   (p->rot_dims == 0 || p->inv_freq), "vy_latent_kv_write: rank %d, rot_dim %d, rotated %d (even, <= rot_dim)", p->rank,
               p->rot_dim, p->rot_dims);
  VY_CHECK_ARG(p->x && p->weight && p->pool && p->pool_row >= p->rank + p->rot_dim && dtype_ok(p->x_dtype) && dtype_ok(p->w_dtype) &&
                   dtype_ok(p->pool_dtype), "vy_latent_kv_write: bad tensors");
  LatDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.table = p->block_table; d.tw = p->table_width; d.bs = p->block_size;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.rank = p->rank; d.rot_dim = p->rot_dim; d.rot_dims = p->rot_dims;
  d.inv_freq = p->inv_freq; d.rot_scale = p->rot_scale == 0.f ? 1.f : p->rot_scale;
  d.w = p->weight; d.w_dt = p->w_dtype; d.eps = p->eps;
  d.pool = p->pool; d.pool_row = p->pool_row; d.pool_dt = p->pool_dtype;
  VY_CHECK_ARG(!p->copy || (dtype_ok(p->copy_dtype) && p->ld_copy >= p->rank + p->rot_dim), "vy_latent_kv_write: bad copy");
  d.copy = p->copy; d.ld_copy = p->ld_copy; d.copy_dt = p->copy_dtype;
  const int gx = (p->max_new + 3) / 4 < 4096 ? (p->max_new + 3) / 4 : 4096;
  VY_CUDA_OK(launch_kernel(latent_kv_write_kernel, dim3(gx, p->n_seqs), dim3(128), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_rope_split(const VyRopeSplit* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_rope_split: null params");
  VY_NEED_DEVICE("vy_rope_split");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0, "vy_rope_split: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->pass >= 0 && p->rot_dim >= 0 && p->rot_dims >= 0 && p->rot_dims <= p->rot_dim && p->rot_dims % 2 == 0 &&
                   (p->rot_dims == 0 || p->inv_freq), "vy_rope_split: heads %d, pass %d, rot_dim %d, rotated %d (even, <= rot_dim)", p->heads,
               p->pass, p->rot_dim, p->rot_dims);
  VY_CHECK_ARG(p->x && dtype_ok(p->x_dtype) && (p->rot_dim == 0 || (p->rot_out && dtype_ok(p->rot_dtype))) &&
                   (!p->pass_out || dtype_ok(p->pass_dtype)), "vy_rope_split: bad tensors");
  SplitDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.heads = p->heads; d.pass = p->pass; d.rot_dim = p->rot_dim; d.rot_dims = p->rot_dims;
  d.inv_freq = p->inv_freq; d.rot_scale = p->rot_scale == 0.f ? 1.f : p->rot_scale;
  d.pass_out = p->pass > 0 ? p->pass_out : nullptr; d.ld_pass = p->ld_pass; d.pass_dt = p->pass_dtype;
  d.rot_out = p->rot_out; d.ld_rot = p->ld_rot; d.rot_head = p->rot_head; d.rot_col = p->rot_col; d.rot_dt = p->rot_dtype;
  const int gx = p->max_new < 4096 ? p->max_new : 4096;
  VY_CUDA_OK(launch_kernel(rope_split_kernel, dim3(gx, p->n_seqs), dim3(128), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_moe_route(const VyMoeRoute* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_moe_route: null params");
  VY_NEED_DEVICE("vy_moe_route");
  VY_CHECK_ARG(p->rows > 0 && p->experts > 0 && p->experts <= 1024 && p->top > 0 && p->top <= p->experts,
               "vy_moe_route: rows %lld, experts %d (<= 1024), top %d", static_cast<long long>(p->rows), p->experts, p->top);
  VY_CHECK_ARG(p->logits && p->ld_logits >= p->experts && p->idx && p->weight, "vy_moe_route: bad tensors");
  RouteDev d;
  d.rows = p->rows; d.experts = p->experts; d.top = p->top;
  d.logits = p->logits; d.ld = p->ld_logits; d.scale = p->scale;
  d.idx = p->idx; d.weight = p->weight; d.dense = p->dense;
  d.kind = p->kind; d.raw = p->raw_weights;
  d.groups = p->groups > 1 ? p->groups : 0; d.keep_groups = d.groups ? p->keep_groups : 0;
  VY_CHECK_ARG(p->kind == VY_ROUTE_SIGMOID || p->kind == VY_ROUTE_SOFTMAX, "vy_moe_route: unknown kind %d", p->kind);
  VY_CHECK_ARG(d.groups == 0 || (p->experts % d.groups == 0 && d.keep_groups > 0 && d.keep_groups <= d.groups &&
                                 p->top <= d.keep_groups * (p->experts / d.groups)),
               "vy_moe_route: %d groups must divide %d experts, keep %d of them, top %d within the kept groups", p->groups, p->experts,
               p->keep_groups, p->top);
  const long long blocks = (p->rows + ROUTE_WARPS - 1) / ROUTE_WARPS;
  VY_CHECK_ARG(blocks <= 2147483647LL, "vy_moe_route: too many rows");
  VY_CUDA_OK(launch_kernel(moe_route_kernel, dim3(static_cast<unsigned>(blocks)), dim3(ROUTE_WARPS * 32),
                           sizeof(float) * ROUTE_WARPS * (p->experts + d.groups), static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_moe_scale(const VyMoeScale* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_moe_scale: null params");
  VY_NEED_DEVICE("vy_moe_scale");
  VY_CHECK_ARG(p->rows > 0 && p->experts >= 0 && p->ff > 0 && p->shared_ff >= 0 && p->experts + p->shared_ff > 0, "vy_moe_scale: bad shape");
  VY_CHECK_ARG(p->h && (p->dense || p->experts == 0) && p->out && dtype_ok(p->h_dtype) && dtype_ok(p->out_dtype), "vy_moe_scale: bad tensors");
  ScaleDev d;
  d.rows = p->rows; d.experts = p->experts; d.ff = p->ff; d.shared_ff = p->shared_ff;
  d.h = p->h; d.ldh = p->ldh; d.h_dt = p->h_dtype;
  d.dense = p->dense; d.sg = p->shared_gate; d.ld_sg = p->ld_gate;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  const int cols = p->experts * p->ff + p->shared_ff;
  VY_CHECK_ARG(p->rows <= 2147483647LL, "vy_moe_scale: too many rows");
  const auto al = [](const void* q, size_t n) { return reinterpret_cast<uintptr_t>(q) % n == 0; };
  const size_t hb = p->h_dtype == VY_F32 ? 32 : 16, ob = p->out_dtype == VY_F32 ? 32 : 16;
  const bool vec = cols % 8 == 0 && p->ldh % 8 == 0 && p->ld_out % 8 == 0 && al(p->h, hb) && al(p->out, ob);
  int gy = (cols + 256 * 8 - 1) / (256 * 8);
  if (gy > 64) gy = 64;
  const dim3 grid(static_cast<unsigned>(p->rows), gy);
  VY_CUDA_OK(vec ? launch_kernel(moe_scale_kernel<true>, grid, dim3(256), 0, static_cast<cudaStream_t>(p->stream), d)
                 : launch_kernel(moe_scale_kernel<false>, grid, dim3(256), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_moe_sort(const VyMoeSort* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_moe_sort: null params");
  VY_NEED_DEVICE("vy_moe_sort");
  VY_CHECK_ARG(p->rows > 0 && p->experts > 0 && p->experts <= 8192 && p->top > 0 && p->rows * p->top <= 2147483647LL, "vy_moe_sort: bad shape");
  VY_CHECK_ARG(p->idx && p->counts && p->offsets && p->perm && p->inv, "vy_moe_sort: bad tensors");
  SortDev d;
  d.pairs = p->rows * p->top; d.experts = p->experts; d.top = p->top;
  d.idx = p->idx; d.counts = p->counts; d.offsets = p->offsets; d.perm = p->perm; d.inv = p->inv;
  VY_CUDA_OK(launch_kernel(moe_sort_kernel, dim3(1), dim3(SORT_T), sizeof(int) * p->experts, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_moe_gather(const VyMoeGather* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_moe_gather: null params");
  VY_NEED_DEVICE("vy_moe_gather");
  VY_CHECK_ARG(p->n > 0 && p->top > 0 && p->width > 0 && p->perm && p->x && p->out && dtype_ok(p->x_dtype) && dtype_ok(p->out_dtype),
               "vy_moe_gather: bad arguments");
  GatherDev d;
  d.n = p->n; d.top = p->top; d.width = p->width; d.perm = p->perm;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  const long long blocks = p->n < 65536 ? p->n : 65536;
  VY_CUDA_OK(launch_kernel(moe_gather_kernel, dim3(static_cast<unsigned>(blocks)), dim3(128), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

extern "C" int vy_moe_combine(const VyMoeCombine* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_moe_combine: null params");
  VY_NEED_DEVICE("vy_moe_combine");
  VY_CHECK_ARG(p->rows > 0 && p->top > 0 && p->width > 0 && p->inv && p->weight && p->part && p->out && dtype_ok(p->part_dtype) &&
                   dtype_ok(p->out_dtype) && (!p->addend || dtype_ok(p->addend_dtype)), "vy_moe_combine: bad arguments");
  CombineDev d;
  d.rows = p->rows; d.top = p->top; d.width = p->width; d.inv = p->inv; d.weight = p->weight;
  d.part = p->part; d.ld_part = p->ld_part; d.part_dt = p->part_dtype;
  d.addend = p->addend; d.ld_addend = p->ld_addend; d.addend_dt = p->addend_dtype;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  const long long blocks = p->rows < 65536 ? p->rows : 65536;
  VY_CUDA_OK(launch_kernel(moe_combine_kernel, dim3(static_cast<unsigned>(blocks)), dim3(128), 0, static_cast<cudaStream_t>(p->stream), d));
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

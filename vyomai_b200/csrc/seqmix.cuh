// Shared by the sequence-mixer kernels (seqmix.cu: token-serial forms used for single tokens and short portions;
// seqmix_tiled.cu: tiled forms used for prompts): activation helpers, the kernels' argument blocks and the tiled launchers.
#pragma once
#include <math.h>

#include "vy_common.cuh"

namespace vy {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float apply_uact(float x, int act) {
  switch (act) {
    case VY_UACT_RELU2: { const float r = fmaxf(x, 0.f); return r * r; }
    case VY_UACT_SILU: return siluf_(x);
    case VY_UACT_SIGMOID: return sigmoidf_(x);
    case VY_UACT_GELU_TANH: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    default: return x;
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float dot4(const float4 a, const float4 b, float acc) {
  acc = fmaf(a.x, b.x, acc);
  acc = fmaf(a.y, b.y, acc);
  acc = fmaf(a.z, b.z, acc);
  return fmaf(a.w, b.w, acc);
}
__device__ __forceinline__ void axpy4(float (&acc)[4], const float a, const float4 x) {
  acc[0] = fmaf(a, x.x, acc[0]);
  acc[1] = fmaf(a, x.y, acc[1]);
  acc[2] = fmaf(a, x.z, acc[2]);
  acc[3] = fmaf(a, x.w, acc[3]);
}
__device__ __forceinline__ const float4& f4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// Rows [0, rows) of a [rows, width] block of `src` into shared memory (row stride ld, zero-filled up to width4 columns, `act`
// applied): row j starts at element off(j) of src, or is all zero when off(j) < 0. Global loads go out in batches of 8 per
// thread before any of them is used, so a tile costs about one memory round trip. vec: src is fp32 and every row start and the
// width are multiples of 4 elements (16-byte loads).
template <int T, typename OffFn>
__device__ __forceinline__ void rows_to_smem(float* dst, int ld, int rows, int width, int width4, const void* src, int dt, bool vec, int act,
                                             OffFn off) {
  constexpr int U = 8;
  if (vec) {
    const int w4 = width4 >> 2, total = rows * w4;
    for (int e0 = threadIdx.x; e0 < total; e0 += T * U) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int e = e0 + u * T;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < total) {
          const int j = e / w4, c = (e - j * w4) << 2;
          const long long o = off(j);
          if (o >= 0 && c < width) v[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + o + c);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int e = e0 + u * T;
        if (e < total) {
          const int j = e / w4, c = (e - j * w4) << 2;
          if (act != VY_UACT_NONE) {
            v[u].x = apply_uact(v[u].x, act); v[u].y = apply_uact(v[u].y, act);
            v[u].z = apply_uact(v[u].z, act); v[u].w = apply_uact(v[u].w, act);
          }
          *reinterpret_cast<float4*>(dst + j * ld + c) = v[u];
        }
      }
    }
  } else {
    const int total = rows * width4;
    for (int e0 = threadIdx.x; e0 < total; e0 += T * U) {
      float v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int e = e0 + u * T;
        v[u] = 0.f;
        if (e < total) {
          const int j = e / width4, c = e - j * width4;
          const long long o = off(j);
          if (o >= 0 && c < width) v[u] = ld_as_float(src, dt, o + c);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int e = e0 + u * T;
        if (e < total) {
          const int j = e / width4, c = e - j * width4;
          dst[j * ld + c] = act != VY_UACT_NONE ? apply_uact(v[u], act) : v[u];
        }
      }
    }
  }
}

// windowed attention with kept first tokens and a sink, over pages
struct WinDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  const void* q; long long ldq; int q_dt;
  const void* kp; const void* vp; int pool_dt;
  long long k_row, v_row;   // row strides of the pools in elements (kv_heads * dim and kv_heads * vdim unless the caller views one pool twice)
  int heads, kv_heads, dim, vdim;
  float scale; int window, keep;
  float out_scale;   // multiplies the normalised output (fp32, before it is rounded to the output dtype)
  int chunk;   // > 0: keys of the query's own block of `chunk` positions only (window and keep are then 0)
  const void* sink; int sink_dt;
  const void* gate; long long ld_gate; int gate_dt;
  void* out; long long ld_out; int out_dt;
};

// One query's visible keys at position pos: [0, nA) (kept first tokens) and [lowB, pos] (the window, or the query's chunk), disjoint
__device__ __forceinline__ void visible_keys(const WinDev& d, int pos, int& nA, int& lowB) {
  if (d.chunk > 0) { nA = 0; lowB = pos / d.chunk * d.chunk; }
  else if (d.window <= 0) { nA = pos + 1; lowB = pos + 1; }
  else { nA = min(d.keep, pos + 1); lowB = max(pos - d.window + 1, nA); }
}

// recurrences (linear attention with a fixed decay, gated delta rule): state [slots, heads, dim, vdim] fp32
struct RecDev {
  const int* cu; const int* pos0; const int* slot;
  const void* q; long long ldq; const void* k; long long ldk; const void* v; long long ldv; int in_dt; int in_act;
  const void* a; long long ld_a; int a_dt;
  const void* b; long long ld_b; int b_dt;
  const void* a_log; int a_log_dt;
  const float* decay;
  int heads, kv_heads, dim, vdim;
  float unit_eps;
  int prepared;   // delta rule: q / k are unit vectors already (q scaled), `a` holds the decays and `b` the write strengths
  float q_scale;  // gated linear attention (the delta kernel without its correction term): multiplies q as it is read
  float* state;
  void* out; long long ld_out; int out_dt;
};

// Prompt-sized steps: defined in seqmix_tiled.cu.
cudaError_t launch_linear_attn_chunked(const RecDev& d, int n_seqs, cudaStream_t st);
cudaError_t launch_window_attn_tiled(const WinDev& d, int n_seqs, int max_new, cudaStream_t st);
// Single tokens whose query heads share key / value rows in groups of 8 or more (latent rows): heads as the rows of a tile.
bool window_attn_heads_applies(const WinDev& d);
long long window_attn_heads_workspace_floats(int n_seqs, int heads, int kv_heads, int vdim);
cudaError_t launch_window_attn_heads(const WinDev& d, int n_seqs, float* ws, long long ws_floats, cudaStream_t st, int* launches);

}  // namespace vy

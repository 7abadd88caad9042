// Prompt-sized forms of two sequence mixers, in fp32 on register tiles (scores, softmax weights, decays and recurrent state
// are 32-bit by the models' definition, so the contractions run on the FMA pipes, not on the 16-bit tensor-core path):
//
//   * linear attention with a fixed decay, chunk by chunk: for a chunk of C tokens with the state S0 before it,
//       O = (Q K^T . D) V + diag(decay^(i+1)) Q S0,   D[i][j] = decay^(i-j) for j <= i, else 0
//       S = decay^C S0 + sum_j decay^(C-1-j) k_j v_j^T
//     one CTA owns (sequence, head, 64 value columns) and walks the chunks in order with its slice of S in shared memory;
//   * windowed softmax attention with kept first tokens and a sink over pages: one CTA owns 64 queries of one head, walks
//     the visible keys in tiles of 64 (the kept prefix first, then the window band) with an online softmax.
//
// Both give the same values as the token-serial kernels of seqmix.cu up to fp32 rounding, whatever the portion sizes.
#include <stdlib.h>

#include "seqmix.cuh"

namespace vy {

// ---- chunked linear attention ------------------------------------------------------------------------------------------
constexpr int LA_C = 64;    // tokens per chunk
constexpr int LA_T = 256;   // threads: a 16 x 16 grid; thread (ti, tj) owns rows ti + 16 r and VS / 16 adjacent value columns
constexpr int LA_LDP = LA_C + 4;

template <int DP, int VS>   // VS: value columns per CTA, 32 (two CTAs per SM, more CTAs) or 64 (less repeated work)
struct LaSmem {
  static constexpr int LDQ = DP + 4;    // row stride of the q / k chunks (floats): rows 1 apart start in distinct 16-byte bank groups
  static constexpr int LDV = VS + 4;    // row stride of the v chunk and the state slice
  static constexpr int floats = 2 * LA_C * LDQ + LA_C * LDV + LA_C * LA_LDP + DP * LDV + LA_C + 4;
};

template <int NV>
__device__ __forceinline__ void ldv(const float* p, float (&x)[NV]) {
  if constexpr (NV == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
    const float2 v = *reinterpret_cast<const float2*>(p);
    x[0] = v.x; x[1] = v.y;
  }
}
template <int NV>
__device__ __forceinline__ void axpyv(float (&acc)[NV], const float a, const float (&x)[NV]) {
#pragma unroll
  for (int e = 0; e < NV; ++e) acc[e] = fmaf(a, x[e], acc[e]);
}

template <int DP, int VS, int OCC>   // OCC: CTAs per SM the register budget is set for
__global__ void __launch_bounds__(LA_T, OCC) linear_attn_chunk_kernel(RecDev d, bool vec) {
  pdl_trigger();
  pdl_wait();
  constexpr int LDQ = LaSmem<DP, VS>::LDQ, LDV = LaSmem<DP, VS>::LDV, LDP = LA_LDP;
  constexpr int NV = VS / 16;               // value columns per thread
  constexpr int DR = DP / 16;               // state rows per thread in the update
  extern __shared__ __align__(16) float la_smem[];
  float* Qs = la_smem;                      // [C][LDQ]
  float* Ks = Qs + LA_C * LDQ;              // [C][LDQ]
  float* Vs = Ks + LA_C * LDQ;              // [C][LDV]
  float* Ps = Vs + LA_C * LDV;              // [C][LDP]
  float* Ss = Ps + LA_C * LDP;              // [DP][LDV]
  float* pw = Ss + DP * LDV;                // decay^n, n = 0 .. C
  const int s = blockIdx.z, h = blockIdx.y, v0 = blockIdx.x * VS;
  const int t = threadIdx.x, ti = t >> 4, tj = t & 15;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (n <= 0) return;
  if (t <= LA_C) pw[t] = static_cast<float>(pow(static_cast<double>(d.decay[h]), static_cast<double>(t)));
  float* sp = d.state + (static_cast<long long>(d.slot[s]) * d.heads + h) * d.dim * d.vdim;
  const bool carried = d.pos0[s] > 0;
  for (int e = t; e < DP * VS; e += LA_T) {
    const int i = e / VS, c = e % VS;
    Ss[i * LDV + c] = (carried && i < d.dim && v0 + c < d.vdim) ? sp[static_cast<long long>(i) * d.vdim + v0 + c] : 0.f;
  }
  for (int t0 = 0; t0 < n; t0 += LA_C) {
    const int nt = min(LA_C, n - t0);
    __syncthreads();
    {
      const long long r0 = base + t0;
      rows_to_smem<LA_T>(Qs, LDQ, LA_C, d.dim, DP, d.q, d.in_dt, vec, d.in_act,
                         [&](int tt) { return tt < nt ? (r0 + tt) * d.ldq + static_cast<long long>(h) * d.dim : -1LL; });
      rows_to_smem<LA_T>(Ks, LDQ, LA_C, d.dim, DP, d.k, d.in_dt, vec, d.in_act,
                         [&](int tt) { return tt < nt ? (r0 + tt) * d.ldk + static_cast<long long>(h) * d.dim : -1LL; });
      rows_to_smem<LA_T>(Vs, LDV, LA_C, min(VS, d.vdim - v0), VS, d.v, d.in_dt, vec, d.in_act,
                         [&](int tt) { return tt < nt ? (r0 + tt) * d.ldv + static_cast<long long>(h) * d.vdim + v0 : -1LL; });
    }
    __syncthreads();
    // one pass over the channels feeds both contractions that read the chunk's queries:
    //   what the earlier chunks left, oi[r][e] = sum_i Q[ti + 16 r][i] S0[i][NV tj + e], and
    //   the weights inside the chunk, P[i][j] = (q_i . k_j) decay^(i-j) for j <= i (rows ti + 16 r, columns tj + 16 c, blocks c <= r)
    float oi[4][NV], p[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
#pragma unroll
      for (int e = 0; e < NV; ++e) oi[r][e] = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) p[r][c] = 0.f;
    }
#pragma unroll (OCC == 1 ? 4 : 2)
    for (int d4 = 0; d4 < DP; d4 += 4) {
      float s0[NV], s1[NV], s2[NV], s3[NV];
      ldv<NV>(Ss + (d4 + 0) * LDV + NV * tj, s0);
      ldv<NV>(Ss + (d4 + 1) * LDV + NV * tj, s1);
      ldv<NV>(Ss + (d4 + 2) * LDV + NV * tj, s2);
      ldv<NV>(Ss + (d4 + 3) * LDV + NV * tj, s3);
      float4 kv[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) kv[c] = f4(Ks + (tj + 16 * c) * LDQ + d4);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float4 qv = f4(Qs + (ti + 16 * r) * LDQ + d4);
        axpyv<NV>(oi[r], qv.x, s0);
        axpyv<NV>(oi[r], qv.y, s1);
        axpyv<NV>(oi[r], qv.z, s2);
        axpyv<NV>(oi[r], qv.w, s3);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (c <= r) p[r][c] = dot4(qv, kv[c], p[r][c]);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = ti + 16 * r, j = tj + 16 * c;
        Ps[i * LDP + j] = (c <= r && j <= i && i < nt) ? p[r][c] * pw[i - j] : 0.f;
      }
    __syncthreads();
    // inside the chunk: oa[r][e] = sum_j P[ti + 16 r][j] V[j][NV tj + e]; row block r only sees j < 16 (r + 1)
    float oa[4][NV];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int e = 0; e < NV; ++e) oa[r][e] = 0.f;
#pragma unroll
    for (int jb = 0; jb < 4; ++jb) {
#pragma unroll
      for (int j4 = 16 * jb; j4 < 16 * jb + 16; j4 += 4) {
        float x0[NV], x1[NV], x2[NV], x3[NV];
        ldv<NV>(Vs + (j4 + 0) * LDV + NV * tj, x0);
        ldv<NV>(Vs + (j4 + 1) * LDV + NV * tj, x1);
        ldv<NV>(Vs + (j4 + 2) * LDV + NV * tj, x2);
        ldv<NV>(Vs + (j4 + 3) * LDV + NV * tj, x3);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          if (r >= jb) {
            const float4 pv = f4(Ps + (ti + 16 * r) * LDP + j4);
            axpyv<NV>(oa[r], pv.x, x0);
            axpyv<NV>(oa[r], pv.y, x1);
            axpyv<NV>(oa[r], pv.z, x2);
            axpyv<NV>(oa[r], pv.w, x3);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = ti + 16 * r;
      if (i < nt) {
        const float wi = pw[i + 1];
        const long long o = static_cast<long long>(base + t0 + i) * d.ld_out + static_cast<long long>(h) * d.vdim + v0 + NV * tj;
#pragma unroll
        for (int e = 0; e < NV; ++e)
          if (v0 + NV * tj + e < d.vdim) st_from_float(d.out, d.out_dt, o + e, fmaf(wi, oi[r][e], oa[r][e]));
      }
    }
    // the state after the chunk: rows ti DR .. ti DR + DR - 1, columns NV tj .. (each thread owns its tile of Ss)
    float sa[DR][NV];
#pragma unroll
    for (int x = 0; x < DR; ++x)
#pragma unroll
      for (int e = 0; e < NV; ++e) sa[x][e] = 0.f;
#pragma unroll 2
    for (int j = 0; j < nt; ++j) {
      const float w = pw[nt - 1 - j];
      float vv[NV];
      ldv<NV>(Vs + j * LDV + NV * tj, vv);
#pragma unroll
      for (int e = 0; e < NV; ++e) vv[e] *= w;
      float kk[DR];
      if constexpr (DR % 4 == 0) {
#pragma unroll
        for (int x = 0; x < DR; x += 4) {
          const float4 k4 = f4(Ks + j * LDQ + ti * DR + x);
          kk[x] = k4.x; kk[x + 1] = k4.y; kk[x + 2] = k4.z; kk[x + 3] = k4.w;
        }
      } else {
#pragma unroll
        for (int x = 0; x < DR; ++x) kk[x] = Ks[j * LDQ + ti * DR + x];
      }
#pragma unroll
      for (int x = 0; x < DR; ++x) axpyv<NV>(sa[x], kk[x], vv);
    }
    const float wc = pw[nt];
#pragma unroll
    for (int x = 0; x < DR; ++x) {
      float* sr = Ss + (ti * DR + x) * LDV + NV * tj;
#pragma unroll
      for (int e = 0; e < NV; ++e) sr[e] = fmaf(wc, sr[e], sa[x][e]);
    }
  }
  __syncthreads();
  for (int e = t; e < DP * VS; e += LA_T) {
    const int i = e / VS, c = e % VS;
    if (i < d.dim && v0 + c < d.vdim) sp[static_cast<long long>(i) * d.vdim + v0 + c] = Ss[i * LDV + c];
  }
}

template <int DP, int VS, int OCC>
static cudaError_t launch_la(const RecDev& d, int n_seqs, cudaStream_t st) {
  constexpr size_t smem = sizeof(float) * LaSmem<DP, VS>::floats;
  static bool once = false;
  if (!once) {
    cudaError_t e = cudaFuncSetAttribute(linear_attn_chunk_kernel<DP, VS, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    once = true;
  }
  const auto al = [](const void* p, long long ld) { return reinterpret_cast<uintptr_t>(p) % 16 == 0 && ld % 4 == 0; };
  const bool vec = d.in_dt == VY_F32 && d.dim % 4 == 0 && d.vdim % 4 == 0 && al(d.q, d.ldq) && al(d.k, d.ldk) && al(d.v, d.ldv);
  return launch_kernel(linear_attn_chunk_kernel<DP, VS, OCC>, dim3((d.vdim + VS - 1) / VS, d.heads, n_seqs), dim3(LA_T), smem, st, d, vec);
}

template <int DP>
static cudaError_t launch_la_dp(const RecDev& d, int n_seqs, cudaStream_t st) {
  // 64-column slices repeat the chunk's q k^T half as often; 32-column slices when those would leave SMs without a CTA
  const long long ctas64 = static_cast<long long>((d.vdim + 63) / 64) * d.heads * n_seqs;
  if (ctas64 >= 148) return launch_la<DP, 64, 1>(d, n_seqs, st);
  const long long ctas32 = static_cast<long long>((d.vdim + 31) / 32) * d.heads * n_seqs;
  // a grid that leaves every CTA an SM of its own gets the whole register file (deeper load / FMA overlap); otherwise two per SM
  return ctas32 <= 148 ? launch_la<DP, 32, 1>(d, n_seqs, st) : launch_la<DP, 32, 2>(d, n_seqs, st);
}

cudaError_t launch_linear_attn_chunked(const RecDev& d, int n_seqs, cudaStream_t st) {
  if (d.dim <= 16) return launch_la_dp<16>(d, n_seqs, st);
  if (d.dim <= 32) return launch_la_dp<32>(d, n_seqs, st);
  if (d.dim <= 64) return launch_la_dp<64>(d, n_seqs, st);
  return launch_la_dp<128>(d, n_seqs, st);   // callers keep dim <= 128 here
}

// ---- tiled windowed attention --------------------------------------------------------------------------------------------
constexpr int WT_M = 64;            // queries per CTA
constexpr int WT_T = 256;           // threads: 16 x 16, each 4 query rows (ti + 16 r) by BN / 16 key columns (tj + 16 c)
// BN: keys per tile. 64 halves the barriers per key; 32 lets two CTAs share an SM at 128-wide heads (the kernel is bound by
// shared-memory and FMA latency with 8 warps, so a second CTA is what fills the issue slots)

template <int MV, int BN>
__global__ void __launch_bounds__(WT_T, BN == 32 ? 2 : 1) window_attn_tiled_kernel(WinDev d, int ldq_s, int ldv_s, int dim4, int vdim4, bool qvec, bool kvvec) {
  pdl_trigger();
  pdl_wait();
  constexpr int WT_N = BN, WT_LDP = BN + 4, NCB = BN / 16;
  extern __shared__ __align__(16) float wt_smem[];
  float* Qs = wt_smem;                       // [WT_M][ldq_s]
  float* Ks = Qs + WT_M * ldq_s;             // [WT_N][ldq_s]
  float* Vs = Ks + WT_N * ldq_s;             // [WT_N][ldv_s]
  float* Ps = Vs + WT_N * ldv_s;             // [WT_M][WT_LDP]
  float* corr_s = Ps + WT_M * WT_LDP;        // [WT_M]
  float* l_s = corr_s + WT_M;                // [WT_M]
  int* kpos_s = reinterpret_cast<int*>(l_s + WT_M);   // [WT_N] key position, -1 past the end
  int* krow_s = kpos_s + WT_N;                        // [WT_N] its row in the pools
  const int s = blockIdx.z, h = blockIdx.y, i0 = blockIdx.x * WT_M;
  const int t = threadIdx.x, ti = t >> 4, tj = t & 15, warp = t >> 5, lane = t & 31;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (i0 >= n) return;
  const int rows = min(WT_M, n - i0);
  const int g = h / (d.heads / d.kv_heads);
  rows_to_smem<WT_T>(Qs, ldq_s, WT_M, d.dim, dim4, d.q, d.q_dt, qvec, VY_UACT_NONE,
               [&](int i) { return i < rows ? static_cast<long long>(base + i0 + i) * d.ldq + static_cast<long long>(h) * d.dim : -1LL; });
  const int p_lo = d.pos0[s] + i0, p_hi = p_lo + rows - 1;
  // visible keys of the tile's queries: [0, nA) (kept first tokens outside the band) and [lo, p_hi] (the band); masks are per pair
  const int lo = d.chunk > 0 ? p_lo / d.chunk * d.chunk : d.window <= 0 ? 0 : max(p_lo - d.window + 1, 0);
  const int nA = d.window <= 0 ? 0 : min(d.keep, lo);
  const int count = nA + (p_hi - lo + 1);
  const int* tab = d.table + static_cast<long long>(s) * d.tw;
  float m[8], l[8];   // softmax statistics of rows 8 warp .. 8 warp + 7, the same in every lane
#pragma unroll
  for (int rr = 0; rr < 8; ++rr) {
    m[rr] = d.sink ? ld_as_float(d.sink, d.sink_dt, h) : -INFINITY;
    l[rr] = d.sink ? 1.f : 0.f;
  }
  float acc[4][MV][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int mm = 0; mm < MV; ++mm)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][mm][e] = 0.f;
  const long long kstride = d.k_row, vstride = d.v_row;
  for (int c0 = 0; c0 < count; c0 += WT_N) {
    __syncthreads();
    if (t < WT_N) {
      const int c = c0 + t;
      const int kp = c < count ? (c < nA ? c : lo + (c - nA)) : -1;
      kpos_s[t] = kp;
      krow_s[t] = kp >= 0 ? tab[kp / d.bs] * d.bs + kp % d.bs : 0;
    }
    __syncthreads();
    rows_to_smem<WT_T>(Ks, ldq_s, WT_N, d.dim, dim4, d.kp, d.pool_dt, kvvec, VY_UACT_NONE,
                 [&](int j) { return kpos_s[j] >= 0 ? static_cast<long long>(krow_s[j]) * kstride + static_cast<long long>(g) * d.dim : -1LL; });
    rows_to_smem<WT_T>(Vs, ldv_s, WT_N, d.vdim, vdim4, d.vp, d.pool_dt, kvvec, VY_UACT_NONE,
                 [&](int j) { return kpos_s[j] >= 0 ? static_cast<long long>(krow_s[j]) * vstride + static_cast<long long>(g) * d.vdim : -1LL; });
    __syncthreads();
    float sc[4][NCB];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < NCB; ++c) sc[r][c] = 0.f;
#pragma unroll 2
    for (int d4 = 0; d4 < dim4; d4 += 4) {
      float4 kv[NCB];
#pragma unroll
      for (int c = 0; c < NCB; ++c) kv[c] = f4(Ks + (tj + 16 * c) * ldq_s + d4);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float4 qv = f4(Qs + (ti + 16 * r) * ldq_s + d4);
#pragma unroll
        for (int c = 0; c < NCB; ++c) sc[r][c] = dot4(qv, kv[c], sc[r][c]);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < NCB; ++c) {
        const int i = ti + 16 * r, j = tj + 16 * c;
        const int p = p_lo + i, kp = kpos_s[j];
        const bool vis = i < rows && kp >= 0 && kp <= p && (d.window <= 0 || p - kp < d.window || kp < d.keep) && (d.chunk <= 0 || kp >= p / d.chunk * d.chunk);
        Ps[i * WT_LDP + j] = vis ? sc[r][c] * d.scale : -INFINITY;
      }
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) {
      float* pr = Ps + (8 * warp + rr) * WT_LDP;
      const float a = pr[lane], b = BN == 64 ? pr[lane + 32] : -INFINITY;
      const float mn = fmaxf(m[rr], warp_max(fmaxf(a, b)));
      const float cr = mn == -INFINITY ? 1.f : expf(m[rr] - mn);
      const float pa = a == -INFINITY ? 0.f : expf(a - mn), pb = b == -INFINITY ? 0.f : expf(b - mn);
      pr[lane] = pa;
      if (BN == 64) pr[lane + 32] = pb;
      l[rr] = fmaf(l[rr], cr, warp_sum(pa + pb));
      m[rr] = mn;
      if (lane == 0) corr_s[8 * warp + rr] = cr;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float cr = corr_s[ti + 16 * r];
#pragma unroll
      for (int mm = 0; mm < MV; ++mm)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][mm][e] *= cr;
    }
    const int nv = min(WT_N, (count - c0 + 3) & ~3);
    for (int j4 = 0; j4 < nv; j4 += 4) {
      float4 pv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) pv[r] = f4(Ps + (ti + 16 * r) * WT_LDP + j4);
#pragma unroll
      for (int mm = 0; mm < MV; ++mm) {
        const int col = 4 * (tj + 16 * mm);
        if (col < vdim4) {
          const float4 x0 = f4(Vs + (j4 + 0) * ldv_s + col), x1 = f4(Vs + (j4 + 1) * ldv_s + col);
          const float4 x2 = f4(Vs + (j4 + 2) * ldv_s + col), x3 = f4(Vs + (j4 + 3) * ldv_s + col);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            axpy4(acc[r][mm], pv[r].x, x0);
            axpy4(acc[r][mm], pv[r].y, x1);
            axpy4(acc[r][mm], pv[r].z, x2);
            axpy4(acc[r][mm], pv[r].w, x3);
          }
        }
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) l_s[8 * warp + rr] = l[rr];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = ti + 16 * r;
    if (i >= rows) continue;
    const long long qrow = base + i0 + i;
    float og = d.out_scale / l_s[i];
    if (d.gate) og *= sigmoidf_(ld_as_float(d.gate, d.gate_dt, qrow * d.ld_gate + h));
#pragma unroll
    for (int mm = 0; mm < MV; ++mm)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = 4 * (tj + 16 * mm) + e;
        if (col < d.vdim) st_from_float(d.out, d.out_dt, qrow * d.ld_out + static_cast<long long>(h) * d.vdim + col, acc[r][mm][e] * og);
      }
  }
}

// ---- single tokens, many query heads per key / value head ---------------------------------------------------------------------
// Latent rows (one key / value head for all query heads) and wide head groups: the heads of ONE token are the query rows of a tile.
// A CTA owns (sequence, 16 heads of one key / value head, one split of the visible keys) and walks its keys 64 at a time: the key
// tile goes to shared memory once (the value tile too, unless values are the leading channels of the key rows), thread (key, 4
// heads) contracts a key row with 4 query rows (no per-pair warp reduction: a lane owns a key), two heads per warp update the
// online softmax, thread (4 heads, every 64th channel) accumulates the output. With several splits the partial (max, sum, output)
// of each goes to a workspace and window_attn_heads_merge_kernel combines them; the sink enters split 0.
constexpr int WH_H = 16, WH_K = 64, WH_T = 256, WH_VC = 4;   // heads and keys per tile, threads, value channels per thread (vdim <= 256)

__global__ void __launch_bounds__(WH_T) window_attn_heads_kernel(WinDev d, int ldk, int ldv, int dim4, int vdim4, bool qvec, bool kvvec, bool alias,
                                                                 int splits, float* ws) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float wh_smem[];
  constexpr int LDS_ = WH_K + 4;
  float* Qs = wh_smem;                       // [WH_H][ldk]
  float* Ks = Qs + WH_H * ldk;               // [WH_K][ldk]
  float* Vs = alias ? Ks : Ks + WH_K * ldk;  // [WH_K][ldv] (alias: the key rows themselves, ldv == ldk)
  float* Ss = (alias ? Ks + WH_K * ldk : Vs + WH_K * ldv);   // [WH_H][LDS_] scores, then weights
  float* corr_s = Ss + WH_H * LDS_;          // [WH_H]
  float* m_s = corr_s + WH_H;                // [WH_H]
  float* l_s = m_s + WH_H;                   // [WH_H]
  int* krow_s = reinterpret_cast<int*>(l_s + WH_H);   // [WH_K] pool row of each key of the tile, -1 past the end
  const int per_kv = d.heads / d.kv_heads, tiles = (per_kv + WH_H - 1) / WH_H;
  const int s = blockIdx.z, g = blockIdx.y / tiles, h0 = g * per_kv + (blockIdx.y % tiles) * WH_H, split = blockIdx.x;
  const int nh = min(WH_H, g * per_kv + per_kv - h0);
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int base = d.cu[s];
  if (d.cu[s + 1] - base <= 0) return;
  const long long qrow = base;
  rows_to_smem<WH_T>(Qs, ldk, WH_H, d.dim, dim4, d.q, d.q_dt, qvec, VY_UACT_NONE,
               [&](int i) { return i < nh ? qrow * d.ldq + static_cast<long long>(h0 + i) * d.dim : -1LL; });
  const int pos = d.pos0[s];
  int nA, lowB;
  visible_keys(d, pos, nA, lowB);
  const int count = nA + (pos + 1 - lowB);
  // this split's keys: tiles of WH_K dealt out in contiguous runs
  const int ktiles = (count + WH_K - 1) / WH_K, tper = (ktiles + splits - 1) / splits;
  const int c_begin = min(split * tper * WH_K, count), c_end = min((split + 1) * tper * WH_K, count);
  const int* tab = d.table + static_cast<long long>(s) * d.tw;
  // softmax statistics of heads 2 warp, 2 warp + 1 (lane-uniform)
  float m[2], l[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int hh = 2 * warp + e;
    const bool sk = d.sink && split == 0 && hh < nh;
    m[e] = sk ? ld_as_float(d.sink, d.sink_dt, h0 + hh) : -INFINITY;
    l[e] = sk ? 1.f : 0.f;
  }
  const int kj = t & 63, hq = t >> 6;   // score phase: key kj, heads 4 hq .. 4 hq + 3; output phase: channels kj + 64 cc, same heads
  float acc[4][WH_VC];
#pragma unroll
  for (int e = 0; e < 4; ++e)
#pragma unroll
    for (int cc = 0; cc < WH_VC; ++cc) acc[e][cc] = 0.f;
  for (int c0 = c_begin; c0 < c_end; c0 += WH_K) {
    __syncthreads();   // the previous tile's readers are done (first pass: Qs is complete after the barrier below)
    if (t < WH_K) {
      const int c = c0 + t;
      int row = -1;
      if (c < c_end) {
        const int kp = c < nA ? c : lowB + (c - nA);
        row = tab[kp / d.bs] * d.bs + kp % d.bs;
      }
      krow_s[t] = row;
    }
    __syncthreads();
    rows_to_smem<WH_T>(Ks, ldk, WH_K, d.dim, dim4, d.kp, d.pool_dt, kvvec, VY_UACT_NONE,
                 [&](int j) { return krow_s[j] >= 0 ? static_cast<long long>(krow_s[j]) * d.k_row + static_cast<long long>(g) * d.dim : -1LL; });
    if (!alias)
      rows_to_smem<WH_T>(Vs, ldv, WH_K, d.vdim, vdim4, d.vp, d.pool_dt, kvvec, VY_UACT_NONE,
                   [&](int j) { return krow_s[j] >= 0 ? static_cast<long long>(krow_s[j]) * d.v_row + static_cast<long long>(g) * d.vdim : -1LL; });
    __syncthreads();
    {
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
      const float* kr = Ks + kj * ldk;
      const float* q0 = Qs + (4 * hq) * ldk;
#pragma unroll 2
      for (int c = 0; c < dim4; c += 4) {
        const float4 k4 = f4(kr + c);
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[e] = dot4(f4(q0 + e * ldk + c), k4, sc[e]);
      }
      const bool vis = krow_s[kj] >= 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) Ss[(4 * hq + e) * LDS_ + kj] = vis ? sc[e] * d.scale : -INFINITY;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float* pr = Ss + (2 * warp + e) * LDS_;
      const float a = pr[lane], b = pr[lane + 32];
      const float mn = fmaxf(m[e], warp_max(fmaxf(a, b)));
      const float cr = mn == -INFINITY ? 1.f : expf(m[e] - mn);
      const float pa = a == -INFINITY ? 0.f : expf(a - mn), pb = b == -INFINITY ? 0.f : expf(b - mn);
      pr[lane] = pa;
      pr[lane + 32] = pb;
      l[e] = fmaf(l[e], cr, warp_sum(pa + pb));
      m[e] = mn;
      if (lane == 0) corr_s[2 * warp + e] = cr;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float cr = corr_s[4 * hq + e];
#pragma unroll
      for (int cc = 0; cc < WH_VC; ++cc) acc[e][cc] *= cr;
    }
    const int nk = min(WH_K, (c_end - c0 + 3) & ~3);
    for (int j4 = 0; j4 < nk; j4 += 4) {
      float4 p4[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) p4[e] = f4(Ss + (4 * hq + e) * LDS_ + j4);
#pragma unroll
      for (int cc = 0; cc < WH_VC; ++cc) {
        const int col = kj + 64 * cc;
        if (col < vdim4) {
          const float v0 = Vs[(j4 + 0) * ldv + col], v1 = Vs[(j4 + 1) * ldv + col], v2 = Vs[(j4 + 2) * ldv + col], v3 = Vs[(j4 + 3) * ldv + col];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a = acc[e][cc];
            a = fmaf(p4[e].x, v0, a);
            a = fmaf(p4[e].y, v1, a);
            a = fmaf(p4[e].z, v2, a);
            a = fmaf(p4[e].w, v3, a);
            acc[e][cc] = a;
          }
        }
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int e = 0; e < 2; ++e) { m_s[2 * warp + e] = m[e]; l_s[2 * warp + e] = l[e]; }
  }
  __syncthreads();
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int hh = 4 * hq + e;
    if (hh >= nh) continue;
    const int h = h0 + hh;
    if (splits == 1) {
      float og = d.out_scale / l_s[hh];
      if (d.gate) og *= sigmoidf_(ld_as_float(d.gate, d.gate_dt, qrow * d.ld_gate + h));
#pragma unroll
      for (int cc = 0; cc < WH_VC; ++cc) {
        const int col = kj + 64 * cc;
        if (col < d.vdim) st_from_float(d.out, d.out_dt, qrow * d.ld_out + static_cast<long long>(h) * d.vdim + col, acc[e][cc] * og);
      }
    } else {
      float* wp = ws + ((static_cast<long long>(s) * d.heads + h) * splits + split) * (d.vdim + 2);
      if (kj == 0) { wp[0] = m_s[hh]; wp[1] = l_s[hh]; }
#pragma unroll
      for (int cc = 0; cc < WH_VC; ++cc) {
        const int col = kj + 64 * cc;
        if (col < d.vdim) wp[2 + col] = acc[e][cc];
      }
    }
  }
}

// combines the splits of one (sequence, head): out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M), times the output gate
__global__ void __launch_bounds__(64) window_attn_heads_merge_kernel(WinDev d, int splits, const float* ws) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y, h = blockIdx.x;
  const int base = d.cu[s];
  if (d.cu[s + 1] - base <= 0) return;
  const float* wp = ws + (static_cast<long long>(s) * d.heads + h) * splits * (d.vdim + 2);
  float M = -INFINITY;
  for (int k = 0; k < splits; ++k) M = fmaxf(M, wp[k * (d.vdim + 2)]);
  float L = 0.f;
  for (int k = 0; k < splits; ++k) {
    const float mk = wp[k * (d.vdim + 2)];
    if (mk != -INFINITY) L = fmaf(wp[k * (d.vdim + 2) + 1], expf(mk - M), L);
  }
  float og = d.out_scale / L;
  const long long qrow = base;
  if (d.gate) og *= sigmoidf_(ld_as_float(d.gate, d.gate_dt, qrow * d.ld_gate + h));
  for (int c = threadIdx.x; c < d.vdim; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < splits; ++k) {
      const float mk = wp[k * (d.vdim + 2)];
      if (mk != -INFINITY) a = fmaf(wp[k * (d.vdim + 2) + 2 + c], expf(mk - M), a);
    }
    st_from_float(d.out, d.out_dt, qrow * d.ld_out + static_cast<long long>(h) * d.vdim + c, a * og);
  }
}

// heads per key / value head from which the heads-as-rows form is used for single tokens
constexpr int WH_MIN_HEADS = 8;

bool window_attn_heads_applies(const WinDev& d) { return d.heads / d.kv_heads >= WH_MIN_HEADS && d.dim <= 256 && d.vdim <= 64 * WH_VC; }

// most splits a launch of this geometry can use: enough CTAs for two per SM, never more than 16
static long long wh_split_bound(int n_seqs, int heads, int kv_heads) {
  const int per_kv = heads / kv_heads, tiles = (per_kv + WH_H - 1) / WH_H;
  const long long ctas = static_cast<long long>(n_seqs) * kv_heads * tiles;
  const long long splits = (2LL * num_sms() + ctas - 1) / ctas;
  return splits > 16 ? 16 : (splits < 1 ? 1 : splits);
}

long long window_attn_heads_workspace_floats(int n_seqs, int heads, int kv_heads, int vdim) {
  const long long splits = wh_split_bound(n_seqs, heads, kv_heads);
  return splits <= 1 ? 0 : static_cast<long long>(n_seqs) * heads * splits * (vdim + 2);
}

cudaError_t launch_window_attn_heads(const WinDev& d, int n_seqs, float* ws, long long ws_floats, cudaStream_t st, int* launches) {
  const int dim4 = (d.dim + 3) & ~3, vdim4 = (d.vdim + 3) & ~3;
  const bool alias = d.vp == d.kp && d.v_row == d.k_row && d.kv_heads == 1 && d.vdim <= d.dim;   // values = leading channels of the key rows
  const int ldk = ((dim4 >> 2) & 1) ? dim4 + 8 : dim4 + 4;   // (row stride / 4) odd: 16-byte reads of rows 1 apart do not collide
  const int ldv = alias ? ldk : vdim4 + 4;                    // rows are filled 16 bytes at a time: a multiple of 4; reads are scalar, consecutive channels
  const size_t floats = static_cast<size_t>(WH_H + WH_K) * ldk + (alias ? 0 : static_cast<size_t>(WH_K) * ldv) + WH_H * (WH_K + 4) + 3 * WH_H;
  const size_t smem = sizeof(float) * floats + sizeof(int) * WH_K;
  const auto al = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool qvec = d.q_dt == VY_F32 && d.dim % 4 == 0 && d.ldq % 4 == 0 && al(d.q);
  const bool kvvec = d.pool_dt == VY_F32 && d.dim % 4 == 0 && d.vdim % 4 == 0 && d.k_row % 4 == 0 && d.v_row % 4 == 0 && al(d.kp) && al(d.vp);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(window_attn_heads_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  const int per_kv = d.heads / d.kv_heads, tiles = (per_kv + WH_H - 1) / WH_H;
  // splits: enough CTAs for two per SM, at most one per 64 keys of the longest possible context, at most 16 and what the workspace holds
  const long long kmax = d.chunk > 0 ? d.chunk : d.window > 0 ? static_cast<long long>(d.window) + d.keep : static_cast<long long>(d.tw) * d.bs;
  long long splits = wh_split_bound(n_seqs, d.heads, d.kv_heads);
  splits = splits < (kmax + WH_K - 1) / WH_K ? splits : (kmax + WH_K - 1) / WH_K;
  if (!ws || ws_floats < static_cast<long long>(n_seqs) * d.heads * splits * (d.vdim + 2)) splits = 1;
  if (splits < 1) splits = 1;
  cudaError_t e = launch_kernel(window_attn_heads_kernel, dim3(static_cast<unsigned>(splits), d.kv_heads * tiles, n_seqs), dim3(WH_T), smem, st, d, ldk,
                                ldv, dim4, vdim4, qvec, kvvec, alias, static_cast<int>(splits), ws);
  *launches = 1;
  if (e != cudaSuccess || splits == 1) return e;
  *launches = 2;
  return launch_kernel(window_attn_heads_merge_kernel, dim3(d.heads, n_seqs), dim3(64), 0, st, d, static_cast<int>(splits), static_cast<const float*>(ws));
}

template <int MV, int BN>
static cudaError_t launch_wt(const WinDev& d, int n_seqs, int max_new, cudaStream_t st) {
  constexpr int WT_N = BN, WT_LDP = BN + 4;
  const int dim4 = (d.dim + 3) & ~3, vdim4 = (d.vdim + 3) & ~3;
  const int ldq_s = ((dim4 >> 2) & 1) ? dim4 + 8 : dim4 + 4;   // (row stride / 4) odd: rows 1 apart start in distinct 16-byte bank groups
  const int ldv_s = vdim4 + 4;
  const size_t smem = sizeof(float) * (static_cast<size_t>(WT_M + WT_N) * ldq_s + static_cast<size_t>(WT_N) * ldv_s + WT_M * WT_LDP + 2 * WT_M) +
                      sizeof(int) * 2 * WT_N;
  const auto al = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool qvec = d.q_dt == VY_F32 && d.dim % 4 == 0 && d.ldq % 4 == 0 && al(d.q);
  const bool kvvec = d.pool_dt == VY_F32 && d.dim % 4 == 0 && d.vdim % 4 == 0 && d.k_row % 4 == 0 && d.v_row % 4 == 0 && al(d.kp) && al(d.vp);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(window_attn_tiled_kernel<MV, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    allowed = smem;
  }
  return launch_kernel(window_attn_tiled_kernel<MV, BN>, dim3((max_new + WT_M - 1) / WT_M, d.heads, n_seqs), dim3(WT_T), smem, st, d, ldq_s, ldv_s,
                       dim4, vdim4, qvec, kvvec);
}

cudaError_t launch_window_attn_tiled(const WinDev& d, int n_seqs, int max_new, cudaStream_t st) {
  static const int bn_env = getenv("VY_WINDOW_ATTN_BN") ? atoi(getenv("VY_WINDOW_ATTN_BN")) : 0;   // development: 32 or 64
  const bool narrow = bn_env ? bn_env == 32 : (d.dim > 64 || d.vdim > 64);   // wide heads: 64-key tiles would take the SM for one CTA
  if (d.vdim <= 64) return narrow ? launch_wt<1, 32>(d, n_seqs, max_new, st) : launch_wt<1, 64>(d, n_seqs, max_new, st);
  if (d.vdim <= 128) return narrow ? launch_wt<2, 32>(d, n_seqs, max_new, st) : launch_wt<2, 64>(d, n_seqs, max_new, st);
  return launch_wt<4, 64>(d, n_seqs, max_new, st);   // vdim <= 256 (checked by the caller): the accumulators leave no room for two CTAs
}

}  // namespace vy

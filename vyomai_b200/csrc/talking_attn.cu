// Attention whose query heads exchange scores before the softmax ("talking heads"), over pages, in fp32:
//   s_h = cap(q_h . k_g(h) * scale),  s_h <- sum_b talk[h, b] s_b,  causal (optionally windowed) mask,
//   softmax with an optional extra term in the denominator (a learned per-head sink, or a sink of score 0),
//   o_h = sum_j w_h[j] v_g(h)[j], times an optional sigmoid gate per head or per channel.
// A head's weights depend on every head's scores of the same (query, key) pair, so a CTA owns ALL heads of its queries:
//   * rows form: one query token per CTA (and one split of its keys). Per tile of 64 keys, for each key/value head the key rows
//     are staged in shared memory once and every query head of the group is contracted with them; the [heads, 64] score block
//     is mixed through `talk` in shared memory, the softmax is online per head, and the value rows are staged and
//     accumulated the same way. Splits write (max, sum, unnormalised output) per head and a merge kernel combines them:
//     single tokens with long contexts fill the GPU although each token is one row.
//   * tiled form (prompts): rows = (head, query) pairs of a tile of TQ queries, 64 or 128 rows by 32 (or 16) keys on a 16 x 16
//     thread grid with register tiles; the key rows of ALL key/value heads are staged per tile, so every thread contracts its
//     rows at once, and the same exchange runs in shared memory between the two contractions.
// Both forms give the same values up to fp32 rounding, whatever the portion sizes.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "seqmix.cuh"

namespace vy {

struct TalkDev {
  const int* cu; const int* pos0; const int* table; int tw, bs;
  const void* q; long long ldq; int q_dt;
  const void* kp; const void* vp; int pool_dt;
  int heads, kv_heads, dim, vdim;
  float scale, softcap; int window;
  const void* talk; int talk_dt;
  const void* sink; int sink_dt; int zero_sink;
  const void* gate; long long ld_gate; int gate_dt; int gate_ch;
  void* out; long long ld_out; int out_dt;
};

// cap * tanh(s / cap) as cap * (1 - 2 / (1 + e^(2 s / cap))): expf and a fast reciprocal, absolute error a few 1e-7 * cap (the softmax
// that follows depends on score differences, i.e. on absolute error); e^x overflowing to inf gives exactly cap, underflow exactly -cap
__device__ __forceinline__ float cap_score(float s, float cap, float two_over_cap) {
  return cap > 0.f ? cap * (1.f - __fdividef(2.f, 1.f + expf(s * two_over_cap))) : s;
}

// the extra softmax term of head h as (score, present)
__device__ __forceinline__ bool sink_of(const TalkDev& d, int h, float& s) {
  if (d.sink) { s = ld_as_float(d.sink, d.sink_dt, h); return true; }
  s = 0.f;
  return d.zero_sink != 0;
}

// talk[h, b] -> T_s[b * Hp + h], zero for the padding heads; identity without a matrix
template <int T>
__device__ __forceinline__ void load_talk(const TalkDev& d, float* T_s, int H, int Hp) {
  for (int e = threadIdx.x; e < H * Hp; e += T) {
    const int b = e / Hp, h = e - b * Hp;
    T_s[e] = h >= H ? 0.f : (d.talk ? ld_as_float(d.talk, d.talk_dt, h * H + b) : (h == b ? 1.f : 0.f));
  }
}

__device__ __forceinline__ int pow2_shift(int n) { return n > 0 && (n & (n - 1)) == 0 ? 31 - __clz(n) : -1; }

__device__ __forceinline__ float gate_of(const TalkDev& d, long long row, int h, int c) {
  if (!d.gate) return 1.f;
  return sigmoidf_(ld_as_float(d.gate, d.gate_dt, row * d.ld_gate + (d.gate_ch ? static_cast<long long>(h) * d.vdim + c : h)));
}

// Stages the rows krow[j] (j < 2^kn_shift; -1 = zero row) of ALL key/value heads into dst[(g * kn + j) * ld + c] (zero-filled up to
// width4 columns): pool rows are [G][width]. Index arithmetic by shifts when width4 / 4 is a power of two (w4_shift >= 0); global
// loads go out in batches of 8 per thread before any of them is used.
template <int T>
__device__ __forceinline__ void stage_heads(float* dst, int ld, int G, int kn_shift, int width, int width4, int w4_shift, const void* src, int dt,
                                            bool vec, const int* krow) {
  constexpr int U = 8;
  const int kn = 1 << kn_shift;
  if (vec) {
    const int w4 = width4 >> 2, total = (G << kn_shift) * w4;
    for (int e0 = threadIdx.x; e0 < total; e0 += T * U) {
      float4 v[U];
      int at[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int e = e0 + u * T;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        at[u] = -1;
        if (e < total) {
          const int jj = w4_shift >= 0 ? e >> w4_shift : e / w4;
          const int c = (e - jj * w4) << 2, g = jj >> kn_shift, j = jj & (kn - 1);
          at[u] = jj * ld + c;
          const int kr = krow[j];
          if (kr >= 0 && c < width)
            v[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + (static_cast<long long>(kr) * G + g) * width + c);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (at[u] >= 0) *reinterpret_cast<float4*>(dst + at[u]) = v[u];
    }
  } else {
    const int total = (G << kn_shift) * width4;
    for (int e0 = threadIdx.x; e0 < total; e0 += T * U) {
      float v[U];
      int at[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int e = e0 + u * T;
        v[u] = 0.f;
        at[u] = -1;
        if (e < total) {
          const int jj = e / width4, c = e - jj * width4, g = jj >> kn_shift, j = jj & (kn - 1);
          at[u] = jj * ld + c;
          const int kr = krow[j];
          if (kr >= 0 && c < width) v[u] = ld_as_float(src, dt, (static_cast<long long>(kr) * G + g) * width + c);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (at[u] >= 0) dst[at[u]] = v[u];
    }
  }
}

// ---- rows form ------------------------------------------------------------------------------------------------------------------
constexpr int TR_T = 256;   // threads

// grid (token of the sequence, sequence, split); kn keys per tile (a power of two from 64 down to 4, by the shared memory they take). Shared memory
// (floats): q [H][dim4] | staged rows [G][kn][ld_s] (keys, then values, of ALL key/value heads) | S [H][kn] | P [H][kn] |
// talk transposed [H][Hp] (Hp = H rounded up to 4, zero padded) | m, l, corr [H] each | acc [H][vdim4] | key rows (int) [kn].
// HB: query heads per thread in the score phase (they share the staged key row): 4 or 2 when the heads per key/value head allow.
template <int HB>
__global__ void __launch_bounds__(TR_T) talk_attn_rows_kernel(TalkDev d, int kn, int dim4, int vdim4, int ld_s, bool qvec, bool kvvec, int splits, float* ws) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float tr_smem[];
  const int H = d.heads, G = d.kv_heads, per = H / G, Hp = (H + 3) & ~3;
  const int kn_shift = 31 - __clz(kn), dsh = pow2_shift(dim4 >> 2), vsh = pow2_shift(vdim4 >> 2);
  float* q_s = tr_smem;
  float* kv_s = q_s + H * dim4;
  float* S_s = kv_s + G * kn * ld_s;
  float* P_s = S_s + H * kn;
  float* T_s = P_s + H * kn;            // T_s[b * Hp + h] = talk[h, b]
  float* acc_s = T_s + H * Hp;          // [H][vdim4]
  float* m_s = acc_s + H * vdim4;
  float* l_s = m_s + H;
  float* c_s = l_s + H;
  int* krow_s = reinterpret_cast<int*>(c_s + H);
  const int s = blockIdx.y, i = blockIdx.x, split = blockIdx.z;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (i >= n) return;
  const long long qrow = base + i;
  const int p = d.pos0[s] + i;
  const int lo = d.window > 0 ? max(p - d.window + 1, 0) : 0;
  const int count = p - lo + 1;
  const int tiles = (count + kn - 1) / kn;
  const int tps = (tiles + splits - 1) / splits;
  const int tile0 = split * tps, tile1 = min(tiles, tile0 + tps);
  const int* tab = d.table + static_cast<long long>(s) * d.tw;
  const float two_over_cap = d.softcap > 0.f ? 2.f / d.softcap : 0.f;

  rows_to_smem<TR_T>(q_s, dim4, H, d.dim, dim4, d.q, d.q_dt, qvec, VY_UACT_NONE,
                     [&](int h) { return qrow * d.ldq + static_cast<long long>(h) * d.dim; });
  load_talk<TR_T>(d, T_s, H, Hp);
  for (int h = t; h < H; h += TR_T) {
    float sk;
    const bool has = splits == 1 && sink_of(d, h, sk);   // with splits the merge adds the sink
    m_s[h] = has ? sk : -INFINITY;
    l_s[h] = has ? 1.f : 0.f;
  }
  for (int e = t; e < H * vdim4; e += TR_T) acc_s[e] = 0.f;

  for (int tile = tile0; tile < tile1; ++tile) {
    const int c0 = tile * kn;
    const int nk = min(kn, count - c0);
    __syncthreads();
    if (t < kn) {
      const int kp = lo + c0 + t;
      krow_s[t] = t < nk ? tab[kp / d.bs] * d.bs + kp % d.bs : -1;
    }
    __syncthreads();
    stage_heads<TR_T>(kv_s, ld_s, G, kn_shift, d.dim, dim4, dsh, d.kp, d.pool_dt, kvvec, krow_s);
    __syncthreads();
    // raw scores: HB heads of one key/value head against one staged key row per thread
    for (int it = t; it < (H / HB) * kn; it += TR_T) {
      const int hb = it >> kn_shift, j = it & (kn - 1), h0 = hb * HB;
      const float* kp = kv_s + ((h0 / per) * kn + j) * ld_s;
      const float* qp = q_s + h0 * dim4;
      float a[HB];
#pragma unroll
      for (int u = 0; u < HB; ++u) a[u] = 0.f;
      for (int c = 0; c < dim4; c += 4) {
        const float4 k4 = f4(kp + c);
#pragma unroll
        for (int u = 0; u < HB; ++u) a[u] = dot4(f4(qp + u * dim4 + c), k4, a[u]);
      }
#pragma unroll
      for (int u = 0; u < HB; ++u) S_s[(h0 + u) * kn + j] = cap_score(a[u] * d.scale, d.softcap, two_over_cap);
    }
    __syncthreads();
    // the value rows replace the keys while the exchange and the softmax run from S_s / P_s
    stage_heads<TR_T>(kv_s, ld_s, G, kn_shift, d.vdim, vdim4, vsh, d.vp, d.pool_dt, kvvec, krow_s);
    for (int it = t; it < (Hp >> 2) * kn; it += TR_T) {   // exchange: 4 receiving heads of one key per thread
      const int hq = it >> kn_shift, j = it & (kn - 1);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int b = 0; b < H; ++b) {
        const float4 w = f4(T_s + b * Hp + 4 * hq);
        const float x = S_s[b * kn + j];
        a.x = fmaf(w.x, x, a.x); a.y = fmaf(w.y, x, a.y); a.z = fmaf(w.z, x, a.z); a.w = fmaf(w.w, x, a.w);
      }
      const bool live = j < nk;
      const int h0 = 4 * hq;
      P_s[h0 * kn + j] = live ? a.x : -INFINITY;
      if (h0 + 1 < H) P_s[(h0 + 1) * kn + j] = live ? a.y : -INFINITY;
      if (h0 + 2 < H) P_s[(h0 + 2) * kn + j] = live ? a.z : -INFINITY;
      if (h0 + 3 < H) P_s[(h0 + 3) * kn + j] = live ? a.w : -INFINITY;
    }
    __syncthreads();
    for (int h = warp; h < H; h += TR_T / 32) {
      float* pr = P_s + h * kn;
      const float a = lane < kn ? pr[lane] : -INFINITY, b = lane + 32 < kn ? pr[lane + 32] : -INFINITY;
      const float mo = m_s[h];
      const float mn = fmaxf(mo, warp_max(fmaxf(a, b)));
      const float cr = mn == -INFINITY ? 1.f : expf(mo - mn);
      const float pa = a == -INFINITY ? 0.f : expf(a - mn), pb = b == -INFINITY ? 0.f : expf(b - mn);
      if (lane < kn) pr[lane] = pa;
      if (lane + 32 < kn) pr[lane + 32] = pb;
      const float sum = warp_sum(pa + pb);
      if (lane == 0) {
        l_s[h] = fmaf(l_s[h], cr, sum);
        m_s[h] = mn;
        c_s[h] = cr;
      }
    }
    __syncthreads();
    // values: 4 adjacent channels of one head per thread, 4 keys per step (weights past the last key are 0, their rows zero-filled)
    const int nk4 = (nk + 3) & ~3, vq = vdim4 >> 2;
    for (int o = t; o < H * vq; o += TR_T) {
      const int h = o / vq, c4 = (o - h * vq) << 2;
      const float* pr = P_s + h * kn;
      const float* vp = kv_s + (h / per) * kn * ld_s + c4;
      float* ap = acc_s + h * vdim4 + c4;
      const float cr = c_s[h];
      float a[4] = {ap[0] * cr, ap[1] * cr, ap[2] * cr, ap[3] * cr};
      for (int j4 = 0; j4 < nk4; j4 += 4) {
        const float4 p4 = f4(pr + j4);
        axpy4(a, p4.x, f4(vp + (j4 + 0) * ld_s));
        axpy4(a, p4.y, f4(vp + (j4 + 1) * ld_s));
        axpy4(a, p4.z, f4(vp + (j4 + 2) * ld_s));
        axpy4(a, p4.w, f4(vp + (j4 + 3) * ld_s));
      }
      *reinterpret_cast<float4*>(ap) = make_float4(a[0], a[1], a[2], a[3]);
    }
  }
  __syncthreads();
  if (splits == 1) {
    for (int o = t; o < H * d.vdim; o += TR_T) {
      const int h = o / d.vdim, c = o - h * d.vdim;
      const float l = l_s[h];
      st_from_float(d.out, d.out_dt, qrow * d.ld_out + o, l > 0.f ? acc_s[h * vdim4 + c] / l * gate_of(d, qrow, h, c) : 0.f);
    }
  } else {
    // part of (row, split): [H] max | [H] sum | [H * vdim] unnormalised output
    float* w = ws + (qrow * splits + split) * static_cast<long long>(H) * (d.vdim + 2);
    for (int h = t; h < H; h += TR_T) {
      w[h] = m_s[h];
      w[H + h] = l_s[h];
    }
    for (int o = t; o < H * d.vdim; o += TR_T) w[2 * H + o] = acc_s[(o / d.vdim) * vdim4 + o % d.vdim];
  }
}

// one CTA per (row, head): combines the splits' parts, adds the sink term, gates and stores
__global__ void __launch_bounds__(64) talk_attn_merge_kernel(TalkDev d, int splits, const float* ws) {
  pdl_trigger();
  pdl_wait();
  const long long row = blockIdx.x;
  const int H = d.heads, h = blockIdx.y;
  const long long part = static_cast<long long>(H) * (d.vdim + 2);
  const float* w0 = ws + row * splits * part;
  float sk;
  const bool has = sink_of(d, h, sk);
  float m = has ? sk : -INFINITY;
  for (int k = 0; k < splits; ++k) m = fmaxf(m, w0[k * part + h]);
  float l = has ? expf(sk - m) : 0.f;
  for (int k = 0; k < splits; ++k) {
    const float mk = w0[k * part + h];
    if (mk != -INFINITY) l = fmaf(w0[k * part + H + h], expf(mk - m), l);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int c = threadIdx.x; c < d.vdim; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < splits; ++k) {
      const float mk = w0[k * part + h];
      if (mk != -INFINITY) a = fmaf(w0[k * part + 2 * H + h * d.vdim + c], expf(mk - m), a);
    }
    st_from_float(d.out, d.out_dt, row * d.ld_out + static_cast<long long>(h) * d.vdim + c, a * inv * gate_of(d, row, h, c));
  }
}

// ---- tiled form -------------------------------------------------------------------------------------------------------------------
// Rows r = h * TQ + i (head h, query i of the tile); RB blocks of 64 rows. Thread (ti, tj) of the 16 x 16 grid owns rows
// 64 b + 4 ti .. + 3 (the same head: TQ is a multiple of 4) and key columns tj (+ 16) in the score phase, and the value
// columns 4 (tj + 16 mm) .. + 3 of those rows in the output phase. Per key tile: the key rows of every key/value head go to
// shared memory ([kv head][key][channel]), each thread contracts its rows with its head's keys, the exchange reads every head's raw
// scores, the online softmax runs by warps over rows, then the value rows replace the keys and are accumulated.
// NT threads (256, or 512 for 256 rows: two CTAs' worth of warps on one staged key tile); a pass of the thread grid covers NT / 4 rows.
template <int NT, int RB, int MV, int KN>   // KN keys per tile: 32, or 16 when many wide key/value heads would not fit otherwise
__global__ void __launch_bounds__(NT, (NT == 256 && RB * MV <= 2) ? 2 : 1)
talk_attn_tiled_kernel(TalkDev d, int TQ, int dim4, int vdim4, int ldq_s, int ldkv, bool qvec, bool kvvec) {
  pdl_trigger();
  pdl_wait();
  constexpr int TT_T = NT, PASS = NT / 4, R = PASS * RB, LDP = KN + 4, NCB = KN / 16;
  extern __shared__ __align__(16) float tt_smem[];
  const int H = d.heads, G = d.kv_heads, per = H / G, Hp = (H + 3) & ~3;
  float* Q_s = tt_smem;                    // [R][ldq_s]
  float* K_s = Q_s + R * ldq_s;            // [G][KN][ldkv]  (keys, then values)
  float* S_s = K_s + G * KN * ldkv;        // [R][LDP] raw scores
  float* P_s = S_s + R * LDP;              // [R][LDP] mixed scores, then weights
  float* T_s = P_s + R * LDP;              // [H][Hp]: T_s[b * Hp + h] = talk[h, b]
  float* corr_s = T_s + H * Hp;            // [R]
  float* m_s = corr_s + R;                 // [R] running maximum
  float* l_s = m_s + R;                    // [R] running sum
  int* krow_s = reinterpret_cast<int*>(l_s + R);   // [KN]
  const int s = blockIdx.y, i0 = blockIdx.x * TQ;
  const int t = threadIdx.x, ti = t >> 4, tj = t & 15, warp = t >> 5, lane = t & 31;
  const int base = d.cu[s], n = d.cu[s + 1] - base;
  if (i0 >= n) return;
  const int nq = min(TQ, n - i0);
  const int rows = H * TQ;   // <= R
  rows_to_smem<TT_T>(Q_s, ldq_s, R, d.dim, dim4, d.q, d.q_dt, qvec, VY_UACT_NONE, [&](int r) {
    const int h = r / TQ, i = r - h * TQ;
    return (r < rows && i < nq) ? static_cast<long long>(base + i0 + i) * d.ldq + static_cast<long long>(h) * d.dim : -1LL;
  });
  load_talk<TT_T>(d, T_s, H, Hp);
  const int p_lo = d.pos0[s] + i0, p_hi = p_lo + nq - 1;
  const int lo = d.window > 0 ? max(p_lo - d.window + 1, 0) : 0;
  const int count = p_hi - lo + 1;
  const int* tab = d.table + static_cast<long long>(s) * d.tw;
  const float two_over_cap = d.softcap > 0.f ? 2.f / d.softcap : 0.f;
  const int dsh = pow2_shift(dim4 >> 2), vsh = pow2_shift(vdim4 >> 2);
  for (int r = t; r < R; r += TT_T) {
    float sk;
    const bool has = r < rows && sink_of(d, r / TQ, sk);
    m_s[r] = has ? sk : -INFINITY;
    l_s[r] = has ? 1.f : 0.f;
  }
  float acc[RB][4][MV][4];
  int kvoff[RB];   // this thread's rows read the staged rows of their key/value head: K_s + kvoff
#pragma unroll
  for (int b = 0; b < RB; ++b) {
    const int r0 = PASS * b + 4 * ti;
    kvoff[b] = r0 < rows ? (r0 / TQ / per) * KN * ldkv : -1;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int mm = 0; mm < MV; ++mm)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[b][r][mm][e] = 0.f;
  }

  for (int c0 = 0; c0 < count; c0 += KN) {
    const int nk = min(KN, count - c0);
    __syncthreads();
    if (t < KN) {
      const int kp = lo + c0 + t;
      krow_s[t] = t < nk ? tab[kp / d.bs] * d.bs + kp % d.bs : -1;
    }
    __syncthreads();
    stage_heads<TT_T>(K_s, ldkv, G, KN == 32 ? 5 : 4, d.dim, dim4, dsh, d.kp, d.pool_dt, kvvec, krow_s);
    __syncthreads();
    // raw scores
#pragma unroll
    for (int b = 0; b < RB; ++b) {
      if (kvoff[b] < 0) continue;
      const int r0 = PASS * b + 4 * ti;
      const float* Kg = K_s + kvoff[b];
      float sc[4][NCB];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < NCB; ++c) sc[r][c] = 0.f;
#pragma unroll 2
      for (int c = 0; c < dim4; c += 4) {
        float4 kv[NCB];
#pragma unroll
        for (int cb = 0; cb < NCB; ++cb) kv[cb] = f4(Kg + (tj + 16 * cb) * ldkv + c);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float4 qv = f4(Q_s + (r0 + r) * ldq_s + c);
#pragma unroll
          for (int cb = 0; cb < NCB; ++cb) sc[r][cb] = dot4(qv, kv[cb], sc[r][cb]);
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int cb = 0; cb < NCB; ++cb) S_s[(r0 + r) * LDP + tj + 16 * cb] = cap_score(sc[r][cb] * d.scale, d.softcap, two_over_cap);
    }
    __syncthreads();
    // values replace the keys while the exchange and the softmax run from S_s / P_s
    stage_heads<TT_T>(K_s, ldkv, G, KN == 32 ? 5 : 4, d.vdim, vdim4, vsh, d.vp, d.pool_dt, kvvec, krow_s);
    // exchange + mask: element (h, i, j) of P = sum_b talk[h, b] S[b, i, j]
    // each thread: 4 receiving heads x one query x 4 keys, reading every head's raw scores of that (query, keys) once
    for (int it = t; it < (Hp >> 2) * TQ * (KN / 4); it += TT_T) {
      const int j4 = (it % (KN / 4)) * 4, hi = it / (KN / 4);
      const int i = hi % TQ, hq = hi / TQ;
      float4 a[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int b = 0; b < H; ++b) {
        const float4 w = f4(T_s + b * Hp + 4 * hq);
        const float4 x = f4(S_s + (b * TQ + i) * LDP + j4);
        a[0].x = fmaf(w.x, x.x, a[0].x); a[0].y = fmaf(w.x, x.y, a[0].y); a[0].z = fmaf(w.x, x.z, a[0].z); a[0].w = fmaf(w.x, x.w, a[0].w);
        a[1].x = fmaf(w.y, x.x, a[1].x); a[1].y = fmaf(w.y, x.y, a[1].y); a[1].z = fmaf(w.y, x.z, a[1].z); a[1].w = fmaf(w.y, x.w, a[1].w);
        a[2].x = fmaf(w.z, x.x, a[2].x); a[2].y = fmaf(w.z, x.y, a[2].y); a[2].z = fmaf(w.z, x.z, a[2].z); a[2].w = fmaf(w.z, x.w, a[2].w);
        a[3].x = fmaf(w.w, x.x, a[3].x); a[3].y = fmaf(w.w, x.y, a[3].y); a[3].z = fmaf(w.w, x.z, a[3].z); a[3].w = fmaf(w.w, x.w, a[3].w);
      }
      const int pq = p_lo + i, kp0 = lo + c0 + j4;
      const bool live = i < nq;
      const auto vis = [&](int kp, int j) { return live && j < nk && kp <= pq && (d.window <= 0 || pq - kp < d.window); };
      const bool v0 = vis(kp0, j4), v1 = vis(kp0 + 1, j4 + 1), v2 = vis(kp0 + 2, j4 + 2), v3 = vis(kp0 + 3, j4 + 3);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int h = 4 * hq + k;
        if (h < H)
          *reinterpret_cast<float4*>(P_s + (h * TQ + i) * LDP + j4) =
              make_float4(v0 ? a[k].x : -INFINITY, v1 ? a[k].y : -INFINITY, v2 ? a[k].z : -INFINITY, v3 ? a[k].w : -INFINITY);
      }
    }
    __syncthreads();
    // online softmax: two adjacent lanes own a row (KN / 2 keys each, 16-byte accesses), one exchange for the maximum and one for the sum
    for (int rb = warp * 16; rb < rows; rb += TT_T / 2) {   // warp-uniform bound: every lane takes part in the exchanges
      constexpr int HK = KN / 2;
      const int r = rb + (lane >> 1);
      const bool live = r < rows;
      float* pr = P_s + (live ? r : rb) * LDP + (t & 1) * HK;
      float x[HK];
#pragma unroll
      for (int k = 0; k < HK; k += 4) {
        const float4 v = f4(pr + k);
        x[k] = v.x; x[k + 1] = v.y; x[k + 2] = v.z; x[k + 3] = v.w;
      }
      float mx = x[0];
#pragma unroll
      for (int k = 1; k < HK; ++k) mx = fmaxf(mx, x[k]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      const float mo = m_s[live ? r : rb];
      const float mn = fmaxf(mo, mx);
      const float cr = mn == -INFINITY ? 1.f : expf(mo - mn);
      float sum = 0.f;
#pragma unroll
      for (int k = 0; k < HK; ++k) {
        x[k] = x[k] == -INFINITY ? 0.f : expf(x[k] - mn);
        sum += x[k];
      }
      if (live) {
#pragma unroll
        for (int k = 0; k < HK; k += 4) *reinterpret_cast<float4*>(pr + k) = make_float4(x[k], x[k + 1], x[k + 2], x[k + 3]);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      __syncwarp();   // both lanes have read m_s[r] before it changes
      if (live && (t & 1) == 0) {
        l_s[r] = fmaf(l_s[r], cr, sum);
        m_s[r] = mn;
        corr_s[r] = cr;
      }
    }
    __syncthreads();
    // values
    const int nv = (nk + 3) & ~3;
#pragma unroll
    for (int b = 0; b < RB; ++b) {
      if (kvoff[b] < 0) continue;
      const int r0 = PASS * b + 4 * ti;
      const float* Vg = K_s + kvoff[b];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float cr = corr_s[r0 + r];
#pragma unroll
        for (int mm = 0; mm < MV; ++mm)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[b][r][mm][e] *= cr;
      }
      for (int j4 = 0; j4 < nv; j4 += 4) {
        float4 pv[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) pv[r] = f4(P_s + (r0 + r) * LDP + j4);
#pragma unroll
        for (int mm = 0; mm < MV; ++mm) {
          const int col = 4 * (tj + 16 * mm);
          if (col < vdim4) {
            const float4 x0 = f4(Vg + (j4 + 0) * ldkv + col), x1 = f4(Vg + (j4 + 1) * ldkv + col);
            const float4 x2 = f4(Vg + (j4 + 2) * ldkv + col), x3 = f4(Vg + (j4 + 3) * ldkv + col);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              axpy4(acc[b][r][mm], pv[r].x, x0);
              axpy4(acc[b][r][mm], pv[r].y, x1);
              axpy4(acc[b][r][mm], pv[r].z, x2);
              axpy4(acc[b][r][mm], pv[r].w, x3);
            }
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < RB; ++b)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = PASS * b + 4 * ti + r;
      if (row >= rows) continue;
      const int h = row / TQ, i = row - h * TQ;
      if (i >= nq) continue;
      const long long qrow = base + i0 + i;
      const float lv = l_s[row];
      const float inv = lv > 0.f ? 1.f / lv : 0.f;
#pragma unroll
      for (int mm = 0; mm < MV; ++mm)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = 4 * (tj + 16 * mm) + e;
          if (col < d.vdim)
            st_from_float(d.out, d.out_dt, qrow * d.ld_out + static_cast<long long>(h) * d.vdim + col, acc[b][r][mm][e] * inv * gate_of(d, qrow, h, col));
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------------------------------------
constexpr int TR_N = 64;   // most keys per tile of the rows form; the split count is planned with it

static int rows_splits(int n_seqs, int max_new, int table_width, int block_size) {
  // single-token steps only: enough CTAs for four per SM (the latency of a tile's loads is hidden by other CTAs), at most one per key tile, at most 64
  if (max_new != 1) return 1;
  const long long rows = static_cast<long long>(n_seqs) * max_new;
  const long long max_tiles = (static_cast<long long>(table_width) * block_size + TR_N - 1) / TR_N;
  long long want = (4 * 148 + rows - 1) / rows;
  if (want > max_tiles) want = max_tiles;
  if (want > 64) want = 64;
  return want < 1 ? 1 : static_cast<int>(want);
}

static size_t rows_smem(const TalkDev& d, int kn, int dim4, int vdim4, int ld_s) {
  const size_t H = d.heads;
  return sizeof(float) * (H * dim4 + static_cast<size_t>(d.kv_heads) * kn * ld_s + 2 * H * kn + H * ((H + 3) & ~3) + 3 * H + H * vdim4) + sizeof(int) * kn;
}

static int pad_ld(int w4) { return ((w4 >> 2) & 1) ? w4 + 8 : w4 + 4; }   // (row stride / 4) odd: rows 1 apart start in distinct 16-byte bank groups

struct TiledPlan { int NT, RB, MV, KN, TQ, ldq_s, ldkv; size_t smem; bool ok; };

static TiledPlan tiled_plan(const TalkDev& d, int dim4, int vdim4) {
  TiledPlan pl;
  memset(&pl, 0, sizeof(pl));
  const int H = d.heads;
  if (d.vdim > 128) return pl;
  pl.MV = d.vdim <= 64 ? 1 : 2;
  // rows per CTA: 64, 128 (256 threads) or 256 (512 threads, each still owning two 4-row blocks): as few as give every head 8 queries
  // per tile, so that each staged key row serves 8 queries of every head of its group
  static const int rows_env = getenv("VY_TALK_ATTN_ROWS") ? atoi(getenv("VY_TALK_ATTN_ROWS")) : 0;   // development: 64, 128 or 256
  if (H * 4 > 256) return pl;
  int R = 64;
  while (R < 256 && (R / H < 8 || H * 4 > R)) R *= 2;
  if ((rows_env == 64 || rows_env == 128 || rows_env == 256) && H * 4 <= rows_env) R = rows_env;
  pl.NT = R == 256 ? 512 : 256;
  pl.RB = R / (pl.NT / 4);
  pl.TQ = (R / H) & ~3;   // queries per tile: a multiple of 4, so the 4 rows of a thread share a head
  pl.ldq_s = pad_ld(dim4);
  pl.ldkv = pad_ld(dim4 > vdim4 ? dim4 : vdim4);
  for (pl.KN = 32; pl.KN >= 16; pl.KN >>= 1) {
    pl.smem = sizeof(float) * (static_cast<size_t>(R) * pl.ldq_s + static_cast<size_t>(d.kv_heads) * pl.KN * pl.ldkv + 2 * static_cast<size_t>(R) * (pl.KN + 4) +
                               static_cast<size_t>(H) * ((H + 3) & ~3) + 3 * R) + sizeof(int) * pl.KN;
    // 32-key tiles when two CTAs fit an SM with them or nothing smaller is needed; 16-key tiles when 32 do not fit at all
    if (pl.smem <= 200 * 1024) { pl.ok = true; break; }
  }
  return pl;
}

template <int NT, int RB, int MV, int KN>
static cudaError_t launch_tiled_kn(const TalkDev& d, const TiledPlan& pl, int n_seqs, int max_new, int dim4, int vdim4, bool qvec, bool kvvec, cudaStream_t st) {
  static size_t allowed = 48 * 1024;
  if (pl.smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(talk_attn_tiled_kernel<NT, RB, MV, KN>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pl.smem));
    if (e != cudaSuccess) return e;
    allowed = pl.smem;
  }
  return launch_kernel(talk_attn_tiled_kernel<NT, RB, MV, KN>, dim3((max_new + pl.TQ - 1) / pl.TQ, n_seqs), dim3(NT), pl.smem, st, d, pl.TQ, dim4, vdim4,
                       pl.ldq_s, pl.ldkv, qvec, kvvec);
}
template <int NT, int RB, int MV>
static cudaError_t launch_tiled(const TalkDev& d, const TiledPlan& pl, int n_seqs, int max_new, int dim4, int vdim4, bool qvec, bool kvvec, cudaStream_t st) {
  return pl.KN == 32 ? launch_tiled_kn<NT, RB, MV, 32>(d, pl, n_seqs, max_new, dim4, vdim4, qvec, kvvec, st)
                     : launch_tiled_kn<NT, RB, MV, 16>(d, pl, n_seqs, max_new, dim4, vdim4, qvec, kvvec, st);
}

}  // namespace vy

#define VY_NEED_DEVICE(name)                                                   \
  if (!vy_device_ok()) {                                                       \
    ::vy::set_error(name ": no sm_100 device (there is no CPU fallback)");     \
    return VY_ERR_NO_DEVICE;                                                   \
  }

extern "C" int64_t vy_talk_attn_workspace_floats(int32_t n_seqs, int32_t max_new, int32_t table_width, int32_t block_size, int32_t heads, int32_t vdim) {
  if (n_seqs <= 0 || max_new <= 0) return 0;
  const int splits = vy::rows_splits(n_seqs, max_new, table_width, block_size);
  if (splits <= 1) return 0;
  return static_cast<int64_t>(n_seqs) * max_new * splits * heads * (vdim + 2);
}

extern "C" int vy_talk_attn(const VyTalkAttn* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_talk_attn: null params");
  VY_NEED_DEVICE("vy_talk_attn");
  VY_CHECK_ARG(p->n_seqs > 0 && p->n_seqs <= 65535 && p->max_new > 0 && p->cu_tokens && p->pos0 && p->block_table && p->block_size > 0 &&
                   p->table_width > 0, "vy_talk_attn: bad batch");
  VY_CHECK_ARG(p->heads > 0 && p->heads <= 1024 && p->kv_heads > 0 && p->heads % p->kv_heads == 0 && p->dim > 0 && p->vdim > 0,
               "vy_talk_attn: heads %d must be a multiple of kv_heads %d; dim %d, vdim %d", p->heads, p->kv_heads, p->dim, p->vdim);
  VY_CHECK_ARG(p->q && p->k_pool && p->v_pool && p->out && dtype_ok(p->q_dtype) && dtype_ok(p->pool_dtype) && dtype_ok(p->out_dtype) &&
                   (!p->talk || dtype_ok(p->talk_dtype)) && (!p->sink || dtype_ok(p->sink_dtype)) && (!p->gate || dtype_ok(p->gate_dtype)),
               "vy_talk_attn: bad tensors");
  TalkDev d;
  d.cu = p->cu_tokens; d.pos0 = p->pos0; d.table = p->block_table; d.tw = p->table_width; d.bs = p->block_size;
  d.q = p->q; d.ldq = p->ldq; d.q_dt = p->q_dtype;
  d.kp = p->k_pool; d.vp = p->v_pool; d.pool_dt = p->pool_dtype;
  d.heads = p->heads; d.kv_heads = p->kv_heads; d.dim = p->dim; d.vdim = p->vdim;
  d.scale = p->scale; d.softcap = p->softcap; d.window = p->window;
  d.talk = p->talk; d.talk_dt = p->talk_dtype;
  d.sink = p->sink; d.sink_dt = p->sink_dtype; d.zero_sink = p->zero_sink;
  d.gate = p->gate; d.ld_gate = p->ld_gate; d.gate_dt = p->gate_dtype; d.gate_ch = p->gate_per_channel;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  const int dim4 = (d.dim + 3) & ~3, vdim4 = (d.vdim + 3) & ~3;
  const auto al = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  const bool qvec = d.q_dt == VY_F32 && d.dim % 4 == 0 && d.ldq % 4 == 0 && al(d.q);
  const bool kvvec = d.pool_dt == VY_F32 && d.dim % 4 == 0 && d.vdim % 4 == 0 && al(d.kp) && al(d.vp);
  const TiledPlan pl = tiled_plan(d, dim4, vdim4);
  VY_CHECK_ARG(p->force_form != 2 || pl.ok, "vy_talk_attn: the tiled form takes heads <= 64 and vdim <= 128 within 200 KB of shared memory");
  const bool tiled = p->force_form == 2 || (p->force_form == 0 && pl.ok && p->max_new >= 8);
  if (tiled) {
    cudaError_t e;
    if (pl.NT == 512) e = pl.MV == 1 ? launch_tiled<512, 2, 1>(d, pl, p->n_seqs, p->max_new, dim4, vdim4, qvec, kvvec, st)
                                     : launch_tiled<512, 2, 2>(d, pl, p->n_seqs, p->max_new, dim4, vdim4, qvec, kvvec, st);
    else if (pl.RB == 1) e = pl.MV == 1 ? launch_tiled<256, 1, 1>(d, pl, p->n_seqs, p->max_new, dim4, vdim4, qvec, kvvec, st)
                                        : launch_tiled<256, 1, 2>(d, pl, p->n_seqs, p->max_new, dim4, vdim4, qvec, kvvec, st);
    else e = pl.MV == 1 ? launch_tiled<256, 2, 1>(d, pl, p->n_seqs, p->max_new, dim4, vdim4, qvec, kvvec, st)
                        : launch_tiled<256, 2, 2>(d, pl, p->n_seqs, p->max_new, dim4, vdim4, qvec, kvvec, st);
    VY_CUDA_OK(e);
    VY_LAUNCH_OK();
    count_launch();
    return VY_OK;
  }
  const int ld_s = pad_ld(dim4 > vdim4 ? dim4 : vdim4);
  // keys per tile: 64 when two CTAs still share an SM, else the most that fit
  static const int kn_env = getenv("VY_TALK_ATTN_KN") ? atoi(getenv("VY_TALK_ATTN_KN")) : 0;   // development: 64, 32 or 16
  int kn = kn_env == 32 || kn_env == 16 ? kn_env : TR_N;
  while (kn > 16 && rows_smem(d, kn, dim4, vdim4, ld_s) > 110 * 1024) kn >>= 1;
  if (rows_smem(d, kn, dim4, vdim4, ld_s) > 110 * 1024) {
    kn = TR_N;
    while (kn > 4 && rows_smem(d, kn, dim4, vdim4, ld_s) > 220 * 1024) kn >>= 1;   // many wide key/value heads: few keys per tile, still exact
  }
  const size_t smem = rows_smem(d, kn, dim4, vdim4, ld_s);
  VY_CHECK_ARG(smem <= 220 * 1024, "vy_talk_attn: %d heads of %d / %d channels need %zu bytes of shared memory per CTA (at most 220 KB)", d.heads, d.dim,
               d.vdim, smem);
  const int per = d.heads / d.kv_heads;
  const int hb = per % 4 == 0 ? 4 : per % 2 == 0 ? 2 : 1;
  auto kern = hb == 4 ? talk_attn_rows_kernel<4> : hb == 2 ? talk_attn_rows_kernel<2> : talk_attn_rows_kernel<1>;
  static size_t allowed[3] = {48 * 1024, 48 * 1024, 48 * 1024};
  if (smem > allowed[hb >> 1]) {
    VY_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    allowed[hb >> 1] = smem;
  }
  int splits = rows_splits(p->n_seqs, p->max_new, p->table_width, p->block_size);
  const long long rows_bound = static_cast<long long>(p->n_seqs) * p->max_new;
  if (splits > 1) {
    const long long need = rows_bound * splits * d.heads * (d.vdim + 2);
    if (!p->workspace || p->workspace_floats < need) splits = 1;   // no scratch given: every query walks all its keys in one CTA
  }
  VY_CUDA_OK(launch_kernel(kern, dim3(p->max_new, p->n_seqs, splits), dim3(TR_T), smem, st, d, kn, dim4, vdim4, ld_s, qvec, kvvec, splits,
                           p->workspace));
  VY_LAUNCH_OK();
  count_launch();
  if (splits > 1) {   // single-token steps: row s is sequence s
    VY_CUDA_OK(launch_kernel(talk_attn_merge_kernel, dim3(static_cast<unsigned>(p->n_seqs), d.heads), dim3(64), 0, st, d, splits,
                             static_cast<const float*>(p->workspace)));
    VY_LAUNCH_OK();
    count_launch();
  }
  return VY_OK;
}

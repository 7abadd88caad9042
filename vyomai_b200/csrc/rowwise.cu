// Row-wise activations over packed rows. vy_poly_norm: a polynomial of the row's normalised powers,
//   out = a N(z) + b N(z^2) + c3 N(z^3) + e,   N(u) = u / sqrt(mean(u^2) + eps) over the row,
// with all statistics and the polynomial in fp32. One CTA per row: the row is read once into shared memory while the sums of
// z^2, z^4 and z^6 are taken, then written from there.
#include <math.h>

#include "seqmix.cuh"

namespace vy {

struct PolyDev {
  long long rows; int width;
  const void* x; long long ldx; int x_dt;
  float a, b, c3, e, eps;
  void* out; long long ld_out; int out_dt;
};

template <int T>
__global__ void __launch_bounds__(T) poly_norm_kernel(PolyDev d) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float pn_row[];
  __shared__ float part[3][T / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long r = blockIdx.x; r < d.rows; r += gridDim.x) {
    const long long xo = r * d.ldx;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int c = threadIdx.x; c < d.width; c += T) {
      const float z = ld_as_float(d.x, d.x_dt, xo + c);
      pn_row[c] = z;
      const float z2 = z * z, z4 = z2 * z2;
      s2 += z2;
      s4 += z4;
      s6 = fmaf(z4, z2, s6);
    }
    s2 = warp_sum(s2);
    s4 = warp_sum(s4);
    s6 = warp_sum(s6);
    __syncthreads();   // the previous row's readers of `part` are done
    if (lane == 0) { part[0][warp] = s2; part[1][warp] = s4; part[2][warp] = s6; }
    __syncthreads();
    s2 = s4 = s6 = 0.f;
#pragma unroll
    for (int w = 0; w < T / 32; ++w) { s2 += part[0][w]; s4 += part[1][w]; s6 += part[2][w]; }
    const float n = static_cast<float>(d.width);
    const float k1 = d.a / sqrtf(s2 / n + d.eps), k2 = d.b / sqrtf(s4 / n + d.eps), k3 = d.c3 / sqrtf(s6 / n + d.eps);
    const long long oo = r * d.ld_out;
    for (int c = threadIdx.x; c < d.width; c += T) {
      const float z = pn_row[c];
      st_from_float(d.out, d.out_dt, oo + c, fmaf(z, fmaf(z, fmaf(z, k3, k2), k1), d.e));
    }
  }
}

}  // namespace vy

#define VY_NEED_DEVICE(name)                                                   \
  if (!vy_device_ok()) {                                                       \
    ::vy::set_error(name ": no sm_100 device (there is no CPU fallback)");     \
    return VY_ERR_NO_DEVICE;                                                   \
  }

extern "C" int vy_poly_norm(const VyPolyNorm* p) {
  using namespace vy;
  VY_CHECK_ARG(p != nullptr, "vy_poly_norm: null params");
  VY_NEED_DEVICE("vy_poly_norm");
  VY_CHECK_ARG(p->rows > 0 && p->width > 0 && p->width <= 49152, "vy_poly_norm: rows %lld, width %d (<= 49152)", static_cast<long long>(p->rows), p->width);
  VY_CHECK_ARG(p->x && p->out && dtype_ok(p->x_dtype) && dtype_ok(p->out_dtype), "vy_poly_norm: bad tensors");
  PolyDev d;
  d.rows = p->rows; d.width = p->width;
  d.x = p->x; d.ldx = p->ldx; d.x_dt = p->x_dtype;
  d.a = p->a; d.b = p->b; d.c3 = p->c3; d.e = p->e; d.eps = p->eps;
  d.out = p->out; d.ld_out = p->ld_out; d.out_dt = p->out_dtype;
  const size_t smem = sizeof(float) * p->width;
  cudaStream_t st = static_cast<cudaStream_t>(p->stream);
  const unsigned blocks = static_cast<unsigned>(p->rows < 1048576 ? p->rows : 1048576);
  if (p->width <= 1024) {
    VY_CUDA_OK(launch_kernel(poly_norm_kernel<128>, dim3(blocks), dim3(128), smem, st, d));
  } else {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
      VY_CUDA_OK(cudaFuncSetAttribute(poly_norm_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      allowed = smem;
    }
    VY_CUDA_OK(launch_kernel(poly_norm_kernel<512>, dim3(blocks), dim3(512), smem, st, d));
  }
  VY_LAUNCH_OK();
  count_launch();
  return VY_OK;
}

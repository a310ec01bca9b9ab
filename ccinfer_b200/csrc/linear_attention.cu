// Gated linear attention: the inputs of the recurrence  S <- diag(alpha_t) S + k_t v_t^T,  o_t = S^T q_t.
//
// The recurrence itself is the plain form of the kernel in delta_rule.cu (ccb_gated_linear_recurrence); this
// file makes its float rows from the projections of a step:
//   q * q_mult, k, v              as they come from the product, in float
//   alpha = sigmoid(z)^(1 / tau)  with z = a + bias per head and key channel, evaluated as
//                                 exp(log sigmoid(z) / tau) with log sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
// Everything here is float; only the loads see the storage type.
#include "common.cuh"

using namespace ccb;

namespace {

// proj [T, ld]: q at oq and k at ok (H * dk each), v at ov (H * dv); a [T, lda]: H * dk decay pre-activations.
template <typename T>
__global__ void __launch_bounds__(256)
gla_prepare_kernel(const T* __restrict__ proj, int ld, int oq, int ok, int ov, const T* __restrict__ a, int lda,
                   const float* __restrict__ bias, float* __restrict__ qn, float* __restrict__ kn,
                   float* __restrict__ vv, float* __restrict__ gg, int rows, int H, int dk, int dv, float q_mult,
                   float inv_tau) {
  ccb::pdl_begin();
  const int qk = H * dk, vw = H * dv;
  const int per_row = 3 * qk + vw;
  const size_t total = (size_t)rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row;
    int c = (int)(i - t * per_row);
    const T* row = proj + t * ld;
    if (c < qk) {
      qn[t * qk + c] = to_f32(row[oq + c]) * q_mult;
    } else if ((c -= qk) < qk) {
      kn[t * qk + c] = to_f32(row[ok + c]);
    } else if ((c -= qk) < qk) {
      const float z = to_f32(a[t * lda + c]) + (bias ? bias[c] : 0.f);
      const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
      gg[t * qk + c] = expf(ls * inv_tau);
    } else {
      c -= qk;
      vv[t * vw + c] = to_f32(row[ov + c]);
    }
  }
}

// The same, four neighbouring channels a thread (every width, offset and stride a multiple of 4, 16-byte bases).
template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

__device__ __forceinline__ float decay_of(float z, float inv_tau) {
  return expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau);
}

template <typename T>
__global__ void __launch_bounds__(256)
gla_prepare_vec_kernel(const T* __restrict__ proj, int ld, int oq, int ok, int ov, const T* __restrict__ a, int lda,
                       const float* __restrict__ bias, float* __restrict__ qn, float* __restrict__ kn,
                       float* __restrict__ vv, float* __restrict__ gg, int rows, int H, int dk, int dv, float q_mult,
                       float inv_tau) {
  ccb::pdl_begin();
  const int qk = H * dk, vw = H * dv;
  const int per_row = (3 * qk + vw) >> 2;
  const size_t total = (size_t)rows * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row;
    int c = (int)(i - t * per_row) * 4;
    const T* row = proj + t * ld;
    if (c < qk) {
      const float4 x = ld4<T>(row + oq + c);
      *reinterpret_cast<float4*>(qn + t * qk + c) = make_float4(x.x * q_mult, x.y * q_mult, x.z * q_mult, x.w * q_mult);
    } else if ((c -= qk) < qk) {
      *reinterpret_cast<float4*>(kn + t * qk + c) = ld4<T>(row + ok + c);
    } else if ((c -= qk) < qk) {
      float4 z = ld4<T>(a + t * lda + c);
      if (bias) {
        const float4 b = *reinterpret_cast<const float4*>(bias + c);
        z.x += b.x; z.y += b.y; z.z += b.z; z.w += b.w;
      }
      *reinterpret_cast<float4*>(gg + t * qk + c) =
          make_float4(decay_of(z.x, inv_tau), decay_of(z.y, inv_tau), decay_of(z.z, inv_tau), decay_of(z.w, inv_tau));
    } else {
      c -= qk;
      *reinterpret_cast<float4*>(vv + t * vw + c) = ld4<T>(row + ov + c);
    }
  }
}

}  // namespace

CCB_API int ccb_gla_prepare(const void* proj, int ld, int oq, int ok, int ov, const void* a, int lda,
                            const float* bias, float* qn, float* kn, float* vv, float* gg, int rows, int H, int dk,
                            int dv, float q_mult, float tau, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || !(tau > 0.f)) return CCB_REFUSE_SIZE;
  if (dtype != CCB_F32 && dtype != CCB_BF16) return CCB_REFUSE_DTYPE;
  const uintptr_t bases = reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(a) |
                          reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(qn) |
                          reinterpret_cast<uintptr_t>(kn) | reinterpret_cast<uintptr_t>(vv) |
                          reinterpret_cast<uintptr_t>(gg);
  if (((H * dk) | (H * dv) | ld | lda | oq | ok | ov) % 4 == 0 && (bases & 15) == 0) {
    const size_t total4 = (size_t)rows * ((3 * H * dk + H * dv) / 4);
    const int blocks4 = (int)((total4 + 255) / 256 < 65535 * 8 ? (total4 + 255) / 256 : 65535 * 8);
    if (dtype == CCB_F32)
      ccb_launch(gla_prepare_vec_kernel<float>, dim3(blocks4), dim3(256), 0, stream, (const float*)proj, ld, oq, ok, ov,
                 (const float*)a, lda, bias, qn, kn, vv, gg, rows, H, dk, dv, q_mult, 1.0f / tau);
    else
      ccb_launch(gla_prepare_vec_kernel<__nv_bfloat16>, dim3(blocks4), dim3(256), 0, stream,
                 (const __nv_bfloat16*)proj, ld, oq, ok, ov, (const __nv_bfloat16*)a, lda, bias, qn, kn, vv, gg, rows, H,
                 dk, dv, q_mult, 1.0f / tau);
    return ccb_launch_status();
  }
  const size_t total = (size_t)rows * (3 * H * dk + H * dv);
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  if (dtype == CCB_F32)
    ccb_launch(gla_prepare_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)proj, ld, oq, ok, ov,
               (const float*)a, lda, bias, qn, kn, vv, gg, rows, H, dk, dv, q_mult, 1.0f / tau);
  else if (dtype == CCB_BF16)
    ccb_launch(gla_prepare_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)proj, ld,
               oq, ok, ov, (const __nv_bfloat16*)a, lda, bias, qn, kn, vv, gg, rows, H, dk, dv, q_mult, 1.0f / tau);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// Mixture of experts: the router's choice, and the activation of the experts' first products.
//
// Router (float throughout): s = softmax(z) over all experts; choice scores c = s + correction; the experts
// form `groups` equal groups of neighbours, a group's score is its largest c, only experts of the `keep` best
// groups can be chosen (the others count as minus infinity); the `top` largest c are chosen (ties: the lower
// index); the weight of a chosen expert is its s, not renormalised.
//
//   moe_route      a warp per token: idx [T, top] (int32, in the order chosen), wts [T, top], and the same as a
//                  dense row dense_w [T, E] (s where chosen, else 0)
//   moe_dense_act  for the form that runs every expert on every token as ONE product over all experts' rows:
//                  act[t, e * F + f] = relu(u)^2 * dense_w[t, e]; the columns after the experts (a shared expert,
//                  weight 1) get relu(u)^2
#include "common.cuh"
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kRouteWarps = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) v = ov, i = oi;
  }
}

// shared memory per warp: s[E], c[E], gs[groups]
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const float* __restrict__ logits, int ldl, const float* __restrict__ correction,
                 int* __restrict__ idx, float* __restrict__ wts, float* __restrict__ dense_w, int rows, int E,
                 int groups, int keep, int top) {
  ccb::pdl_begin();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= rows) return;
  float* s = smem + (size_t)warp * (2 * E + groups);
  float* c = s + E;
  float* gs = c + E;
  const float* z = logits + (size_t)t * ldl;
  float mx = -CUDART_INF_F;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = expf(z[e] - mx);
    s[e] = v;
    sum += v;
  }
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) {
    s[e] = s[e] / sum;
    c[e] = s[e] + (correction ? correction[e] : 0.f);
    if (dense_w) dense_w[(size_t)t * E + e] = 0.f;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int gsz = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float m = -CUDART_INF_F;
      for (int j = 0; j < gsz; ++j) m = fmaxf(m, c[g * gsz + j]);
      gs[g] = m;
    }
    __syncwarp();
    // the best `keep` groups are marked by +inf in gs, one at a time
    for (int k = 0; k < keep; ++k) {
      float v = -CUDART_INF_F;
      int i = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] != CUDART_INF_F && (gs[g] > v || i == 0x7fffffff)) v = gs[g], i = g;
      warp_argmax(v, i);
      if (lane == 0) gs[i] = CUDART_INF_F;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / gsz] != CUDART_INF_F) c[e] = -CUDART_INF_F;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float v = -CUDART_INF_F;
    int i = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float ce = c[e];
      if (!isnan(ce) && ce != CUDART_INF_F && (ce > v || i == 0x7fffffff)) v = ce, i = e;   // +inf marks a taken one
    }
    warp_argmax(v, i);
    if (lane == 0) {
      idx[(size_t)t * top + k] = i;
      wts[(size_t)t * top + k] = s[i];
      if (dense_w) dense_w[(size_t)t * E + i] = s[i];
      c[i] = CUDART_INF_F;
    }
    __syncwarp();
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_dense_act_kernel(T* __restrict__ act, int ld, const float* __restrict__ dense_w, int rows, int E, int F,
                     int shared) {
  ccb::pdl_begin();
  const int width = E * F + shared;
  const size_t total = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    T* p = act + t * ld + c;
    float u = fmaxf(to_f32(*p), 0.f);
    u *= u;
    if (c < E * F) {
      const float w = dense_w[t * E + c / F];
      u = w == 0.f ? 0.f : u * w;   // an expert that was not chosen gives exact zeros
    }
    *p = from_f32<T>(u);
  }
}

}  // namespace

CCB_API int ccb_moe_route(const float* logits, int ldl, const float* correction, int* idx, float* wts,
                          float* dense_w, int rows, int E, int groups, int keep, int top, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > (E / groups) * keep)
    return CCB_REFUSE_SIZE;
  const size_t smem = (size_t)kRouteWarps * (2 * E + groups) * sizeof(float);
  if (smem > 96 * 1024) return CCB_REFUSE_SIZE;
  cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ccb_launch(moe_route_kernel, dim3((rows + kRouteWarps - 1) / kRouteWarps), dim3(kRouteWarps * 32), smem, stream,
             logits, ldl, correction, idx, wts, dense_w, rows, E, groups, keep, top);
  return ccb_launch_status();
}

CCB_API int ccb_moe_dense_act(void* act, int ld, const float* dense_w, int rows, int E, int F, int shared, int dtype,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E < 0 || F <= 0 || shared < 0 || ld < E * F + shared) return CCB_REFUSE_SIZE;
  const size_t total = (size_t)rows * (E * F + shared);
  const int blocks = (int)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
  if (dtype == CCB_F32)
    ccb_launch(moe_dense_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)act, ld, dense_w, rows, E, F,
               shared);
  else if (dtype == CCB_BF16)
    ccb_launch(moe_dense_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)act, ld,
               dense_w, rows, E, F, shared);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

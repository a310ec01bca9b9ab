// Latent attention: softmax attention whose keys and values are all made from ONE low-rank vector per token.
//
// Per token the layer keeps c (rank R, an RMS-normed projection of the input) and kr (r coordinates, rotated by
// the position, shared by all heads).  Head h has  key_j = [Wuk_h c_j | kr_j]  and  value_j = Wuv_h c_j, so
//   score_ij = (qu_i . Wuk_h c_j + qr_i . kr_j) * scale = ((Wuk_h^T qu_i) . c_j + qr_i . kr_j) * scale
//   out_i    = Wuv_h (sum_j p_ij c_j)
// and attention runs over the cached rows [c | kr] themselves, every head reading the same row: the query is
// carried into the latent space first (a product per head, done by the caller), the weighted sum of c comes
// back out through Wuv_h afterwards.  A query at position p sees the keys p - window + 1 .. p.  The softmax has
// one more term per head, exp(sink_h), with no key and no value (it starts the running maximum and sum).
// Each head's result is multiplied by sigmoid(gate logit of the head) before it is written.
//
// Two kernels:
//   latent_prepare    a block per token: c = x / rms(x) * w and kr = rot(x') into the cache row of the token;
//                     the rotated part of every head's query into the query rows [T, H, R + r] (float)
//   latent_attention  a block per (run of `tq` query tokens of a request, group of heads): 32 cached rows at
//                     a time are staged in shared memory as floats; a warp owns one (query, head): a lane
//                     takes a key for the scores, then a slice of the coordinates for the weighted sum
//
// Scores, weights, sums and the rotation are float whatever the storage type.
#include "common.cuh"
#include <math_constants.h>

using namespace ccb;

namespace {

constexpr int kPrepThreads = 128;

// proj [T, ld]: columns q at oq (H heads of [d | r]) and the latent row at oc ([R | r]).
// cache [slots, R + r]; qa [T, H, R + r] float (only the last r of each head are written here).
template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
latent_prepare_kernel(const T* __restrict__ proj, int ld, int oq, int oc, const float* __restrict__ w,
                      const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
                      const int* __restrict__ slot_map, T* __restrict__ cache, int num_slots, float* __restrict__ qa,
                      int H, int d, int r, int R, float eps, int* status) {
  ccb::pdl_begin();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const T* row = proj + (size_t)t * ld;
  const int half = rot_dims >> 1;
  const int slot = slot_map ? slot_map[t] : -1;
  const bool keep = slot >= 0;
  if (keep && slot >= num_slots) set_status(status, CCB_ST_BAD_SLOT);
  if (keep && slot < num_slots) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += kPrepThreads) {
      const float v = to_f32(row[oc + i]);
      ss += v * v;
    }
    ss = block_sum<kPrepThreads>(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    T* dst = cache + (size_t)slot * (R + r);
    for (int i = threadIdx.x; i < R; i += kPrepThreads) dst[i] = from_f32<T>(to_f32(row[oc + i]) * inv * w[i]);
    const T* kr = row + oc + R;
    for (int i = threadIdx.x; i < r; i += kPrepThreads) {
      float v;
      if (i < rot_dims) {
        const int j = i < half ? i : i - half;
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        const float a = to_f32(kr[j]), b = to_f32(kr[j + half]);
        v = i < half ? a * cs - b * sn : b * cs + a * sn;
      } else {
        v = to_f32(kr[i]);
      }
      dst[R + i] = from_f32<T>(v);
    }
  }
  for (int i = threadIdx.x; i < H * r; i += kPrepThreads) {
    const int h = i / r, k = i - h * r;
    const T* qr = row + oq + (size_t)h * (d + r) + d;
    float v;
    if (k < rot_dims) {
      const int j = k < half ? k : k - half;
      float sn, cs;
      sincosf((float)pos * inv_freq[j], &sn, &cs);
      const float a = to_f32(qr[j]), b = to_f32(qr[j + half]);
      v = k < half ? a * cs - b * sn : b * cs + a * sn;
    } else {
      v = to_f32(qr[k]);
    }
    qa[((size_t)t * H + h) * (R + r) + R + k] = v;
  }
}

constexpr int kAttWarps = 8;
constexpr int kKeys = 32;   // cached rows staged at a time

// NV: coordinates of c per lane (R <= 32 NV).
// Shared memory: tile [kKeys][LD] floats (LD odd: a lane per row reads without bank conflicts), then the
// queries of the block's warps [kAttWarps][R + r].
template <typename T, int NV>
__global__ void __launch_bounds__(kAttWarps * 32)
latent_attention_kernel(const float* __restrict__ qa, const T* __restrict__ cache, const float* __restrict__ sink,
                        const T* __restrict__ gate, int ldg, T* __restrict__ out, const int* __restrict__ cu_q,
                        const int* __restrict__ pos0, const int* __restrict__ entry_of_token, const int* __restrict__ block_table, int bt_stride, int entry0,
                        int H, int R, int r, int page_size, int num_pages, int window, float scale, int tq,
                        int* status) {
  ccb::pdl_begin();
  extern __shared__ __align__(16) float smem[];
  const int W = R + r;
  const int LD = W | 1;
  float* tile = smem;
  float* qs = smem + (size_t)kKeys * LD;
  const int e = entry0 + blockIdx.z;
  const int r0 = cu_q[e], n = cu_q[e + 1] - r0;
  const int qbase = blockIdx.x * tq;
  if (qbase >= n || entry_of_token[r0 + qbase] < 0) return;   // (rows that pad a replayed step belong to no request)
  const int hg = kAttWarps / tq;   // heads per block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi = warp / hg, head = blockIdx.y * hg + (warp - qi * hg);
  const bool live = qbase + qi < n && head < H;
  const int p_first = pos0[e] + qbase;
  const int p_last = p_first + min(tq, n - qbase) - 1;
  const int p = p_first + qi;                     // this warp's position
  const int t = r0 + qbase + qi;                  // and token row
  const int j_lo = max(0, p_first - window + 1);
  const int my_lo = max(0, p - window + 1);
  const int* bt = block_table + (size_t)e * bt_stride;

  float* q = qs + (size_t)warp * W;
  if (live) {
    const float* src = qa + ((size_t)t * H + head) * W;
    for (int i = lane; i < W; i += 32) q[i] = src[i];
  }
  float m = live ? sink[head] : 0.f, l = 1.f;   // the sink: one term exp(sink) with no key and no value
  float acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;

  for (int j0 = j_lo & ~(kKeys - 1); j0 <= p_last; j0 += kKeys) {
    __syncthreads();   // the tile of the round before has been read (and, the first time, q is written)
    for (int rr = warp; rr < kKeys; rr += kAttWarps) {
      const int j = j0 + rr;
      float* dst = tile + (size_t)rr * LD;
      const T* src = nullptr;
      if (j >= j_lo && j <= p_last) {
        const int lp = j / page_size;
        const int page = lp < bt_stride ? bt[lp] : -1;
        if (page < 0 || page >= num_pages) set_status(status, CCB_ST_BAD_PAGE);
        else src = cache + ((size_t)page * page_size + (j - lp * page_size)) * W;
      }
      if (src) for (int i = lane; i < W; i += 32) dst[i] = to_f32(src[i]);
      else for (int i = lane; i < W; i += 32) dst[i] = 0.f;
    }
    __syncthreads();
    if (!live) continue;
    const int j = j0 + lane;
    const float* kj = tile + (size_t)lane * LD;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int i = 0;
    for (; i + 3 < W; i += 4) {
      s0 = fmaf(q[i], kj[i], s0);
      s1 = fmaf(q[i + 1], kj[i + 1], s1);
      s2 = fmaf(q[i + 2], kj[i + 2], s2);
      s3 = fmaf(q[i + 3], kj[i + 3], s3);
    }
    for (; i < W; ++i) s0 = fmaf(q[i], kj[i], s0);
    float s = ((s0 + s1) + (s2 + s3)) * scale;
    if (j < my_lo || j > p) s = -CUDART_INF_F;
    const float m_new = fmaxf(m, warp_max(s));   // finite: m starts at the sink
    const float corr = expf(m - m_new);
    const float pj = expf(s - m_new);            // 0 for a key that is not seen
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[v] *= corr;
    for (int k = 0; k < kKeys; ++k) {
      const float pk = __shfl_sync(0xffffffffu, pj, k);
      if (pk == 0.f) continue;                   // the same for every lane
      const float* ck = tile + (size_t)k * LD;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = lane + 32 * v;
        if (c < R) acc[v] = fmaf(pk, ck[c], acc[v]);
      }
    }
  }
  if (!live) return;
  const float g = 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * ldg + head])));
  const float f = g / l;
  T* dst = out + ((size_t)t * H + head) * R;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = lane + 32 * v;
    if (c < R) dst[c] = from_f32<T>(acc[v] * f);
  }
}

template <typename T, int NV>
int launch_attention(const float* qa, const void* cache, const float* sink, const void* gate, int ldg, void* out,
                     const int* cu_q, const int* pos0, const int* eot, const int* block_table, int bt_stride, int entry0, int n_entries,
                     int max_q, int H, int R, int r, int page_size, int num_pages, int window, float scale,
                     int* status, cudaStream_t stream) {
  // a block's warps share the staged rows: first among the heads of one query (they see the same keys), and
  // where a layer has fewer heads than a block has warps, among neighbouring queries too
  int hg = 1;
  while (hg < kAttWarps && hg < H) hg *= 2;
  const int tq = kAttWarps / hg;
  const int W = R + r;
  const size_t smem = ((size_t)kKeys * (W | 1) + (size_t)kAttWarps * W) * sizeof(float);
  if (smem > 200 * 1024) return CCB_REFUSE_SIZE;
  cudaFuncSetAttribute(latent_attention_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((max_q + tq - 1) / tq, (H + hg - 1) / hg, n_entries);
  ccb_launch(latent_attention_kernel<T, NV>, grid, dim3(kAttWarps * 32), smem, stream, qa, (const T*)cache, sink,
             (const T*)gate, ldg, (T*)out, cu_q, pos0, eot, block_table, bt_stride, entry0, H, R, r, page_size,
             num_pages, window, scale, tq, status);
  return ccb_launch_status();
}

template <typename T>
int pick_attention(const float* qa, const void* cache, const float* sink, const void* gate, int ldg, void* out,
                   const int* cu_q, const int* pos0, const int* eot, const int* block_table, int bt_stride, int entry0, int n_entries,
                   int max_q, int H, int R, int r, int page_size, int num_pages, int window, float scale, int* status,
                   cudaStream_t stream) {
#define CCB_LAT(NV)                                                                                              \
  return launch_attention<T, NV>(qa, cache, sink, gate, ldg, out, cu_q, pos0, eot, block_table, bt_stride, entry0, \
                                 n_entries, max_q, H, R, r, page_size, num_pages, window, scale, status, stream)
  if (R <= 32) CCB_LAT(1);
  if (R <= 64) CCB_LAT(2);
  if (R <= 128) CCB_LAT(4);
  if (R <= 256) CCB_LAT(8);
  if (R <= 512) CCB_LAT(16);
  if (R <= 1024) CCB_LAT(32);
#undef CCB_LAT
  return CCB_REFUSE_SIZE;
}

}  // namespace

CCB_API int ccb_latent_prepare(const void* proj, int ld, int oq, int oc, const float* w, const float* inv_freq,
                               int rot_dims, const int* positions, const int* slot_map, void* cache, int num_slots,
                               float* qa, int T, int H, int d, int r, int R, float eps, int dtype, int* status,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || d < 0 || r < 0 || R <= 0 || rot_dims < 0 || rot_dims > r || (rot_dims & 1)) return CCB_REFUSE_SIZE;
  if (rot_dims > 0 && inv_freq == nullptr) return CCB_REFUSE_ARG;
  if (dtype == CCB_F32)
    ccb_launch(latent_prepare_kernel<float>, dim3(T), dim3(kPrepThreads), 0, stream, (const float*)proj, ld, oq, oc, w,
               inv_freq, rot_dims, positions, slot_map, (float*)cache, num_slots, qa, H, d, r, R, eps, status);
  else if (dtype == CCB_BF16)
    ccb_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(kPrepThreads), 0, stream,
               (const __nv_bfloat16*)proj, ld, oq, oc, w, inv_freq, rot_dims, positions, slot_map,
               (__nv_bfloat16*)cache, num_slots, qa, H, d, r, R, eps, status);
  else
    return CCB_REFUSE_DTYPE;
  return ccb_launch_status();
}

// Entries entry0 .. entry0 + n_entries - 1 of the step, none with more than max_q tokens.
CCB_API int ccb_latent_attention(const float* qa, const void* cache, const float* sink, const void* gate, int ldg,
                                 void* out, const int* cu_q, const int* pos0, const int* entry_of_token,
                                 const int* block_table, int bt_stride, int entry0, int n_entries, int max_q, int H, int R, int r, int page_size,
                                 int num_pages, int window, float scale, int dtype, int* status,
                                 cudaStream_t stream) {
  if (n_entries <= 0 || max_q <= 0) return 0;
  if (H <= 0 || R <= 0 || r < 0 || page_size <= 0 || window <= 0 || n_entries > 65535) return CCB_REFUSE_SIZE;
  if (dtype == CCB_F32)
    return pick_attention<float>(qa, cache, sink, gate, ldg, out, cu_q, pos0, entry_of_token, block_table, bt_stride, entry0,
                                 n_entries, max_q, H, R, r, page_size, num_pages, window, scale, status, stream);
  if (dtype == CCB_BF16)
    return pick_attention<__nv_bfloat16>(qa, cache, sink, gate, ldg, out, cu_q, pos0, entry_of_token, block_table, bt_stride, entry0,
                                         n_entries, max_q, H, R, r, page_size, num_pages, window, scale, status,
                                         stream);
  return CCB_REFUSE_DTYPE;
}

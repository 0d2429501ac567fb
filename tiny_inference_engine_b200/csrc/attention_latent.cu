// Attention whose keys and values come from one latent vector per token (and one rotated key part that all heads
// share). What the cache holds per token is the row [c | r]: c the normed latent (rank floats), r the rotated part
// (rot floats). With W_uk and W_uv the per-head maps from c to the unrotated key and to the value,
//
//     score(h, i, j) = scale * ((W_uk_h^T q_plain_h(i)) . c_j + q_rot_h(i) . r_j),    out_h(i) = W_uv_h (sum_j p_ij c_j)
//
// so every head attends over the same rows with a query of rank + rot dimensions and gets back a weighted sum of
// latents: attention with one kv head whose value is the first `rank` elements of its key. The two per-head maps
// are products around the attention (batched over heads); the kernels here are what stands between them:
//
//   latent_prep      one block per token: RMS norm of the query latent (to its own buffer), RMS norm of c and the
//                    rotation of r, both into the key plane at the token's slot.
//   latent_query_rot one warp per (token, head): the rotated part of the head's query into the tail of its folded query.
//   head_gate_mul    y[t, h, :] *= sigmoid(gate[t, h]): one gate per head.
#include <math.h>

#include "common.cuh"

namespace tie {

// angle = float(pos) * inv_freq[i]; pair (i, i + rot/2).
template <typename T>
__global__ void __launch_bounds__(256) latent_prep_kernel(const T* __restrict__ proj, long long stride, int q_off, int q_rank,
                                                          int kv_off, int rank, int rot, const float* __restrict__ wq,
                                                          const float* __restrict__ wkv, float eps,
                                                          const float* __restrict__ inv_freq,
                                                          const int* __restrict__ positions, const int* __restrict__ slots,
                                                          T* __restrict__ cq, T* __restrict__ k_cache) {
  pdl_sync();
  __shared__ float scratch[33];
  const long long t = blockIdx.x;
  const T* row = proj + t * stride;
  // the query latent
  float ss = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = ld(row + q_off + i);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  float inv = 1.0f / sqrtf(ss / static_cast<float>(q_rank) + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) st(cq + t * q_rank + i, (ld(row + q_off + i) * inv) * wq[i]);
  // the key/value latent and the rotated key part
  const int slot = slots[t];
  ss = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = ld(row + kv_off + i);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  if (slot < 0) return;                        // a row that pads a captured batch
  inv = 1.0f / sqrtf(ss / static_cast<float>(rank) + eps);
  T* dst = k_cache + static_cast<long long>(slot) * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) st(dst + i, (ld(row + kv_off + i) * inv) * wkv[i]);
  const float pos = static_cast<float>(positions[t]);
  const int half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float a = pos * inv_freq[i];
    const float c = cosf(a), s = sinf(a);
    const float u = ld(row + kv_off + rank + i), v = ld(row + kv_off + rank + half + i);
    st(dst + rank + i, u * c - v * s);
    st(dst + rank + half + i, v * c + u * s);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) latent_query_rot_kernel(const T* __restrict__ q, long long q_stride, int dim, int rot,
                                                               const float* __restrict__ inv_freq,
                                                               const int* __restrict__ positions, T* __restrict__ folded,
                                                               long long folded_stride, int rank, int heads,
                                                               long long items) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / heads;
  const int h = static_cast<int>(item % heads);
  const T* src = q + t * q_stride + static_cast<long long>(h) * (dim + rot) + dim;
  T* dst = folded + t * folded_stride + static_cast<long long>(h) * (rank + rot) + rank;
  const float pos = static_cast<float>(positions[t]);
  const int half = rot / 2;
  for (int i = lane; i < half; i += 32) {
    const float a = pos * inv_freq[i];
    const float c = cosf(a), s = sinf(a);
    const float u = ld(src + i), v = ld(src + half + i);
    st(dst + i, u * c - v * s);
    st(dst + half + i, v * c + u * s);
  }
}

template <typename T>
__global__ void head_gate_mul_kernel(T* __restrict__ y, long long y_stride, const T* __restrict__ gate, long long gate_stride,
                                     int width, int head_size, long long total) {
  pdl_sync();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / width;
  const int c = static_cast<int>(idx - t * width);
  const float g = ld(gate + t * gate_stride + c / head_size);
  T* p = y + t * y_stride + c;
  st(p, ld(p) * (1.0f / (1.0f + expf(-g))));
}

}  // namespace tie

using namespace tie;

TIE_API int tie_latent_prep(int dtype, const void* proj, long long stride, int q_off, int q_rank, int kv_off, int rank, int rot,
                            const float* wq, const float* wkv, float eps, const float* inv_freq, const int* positions,
                            const int* slots, void* cq, void* k_cache, int tokens, cudaStream_t s) {
  TIE_REQUIRE(q_rank > 0 && rank > 0 && rot >= 0 && rot % 2 == 0, "latent_prep: bad sizes q_rank=%d rank=%d rot=%d", q_rank, rank, rot);
  if (tokens <= 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((latent_prep_kernel<float>), tokens, 256, 0, s, static_cast<const float*>(proj), stride, q_off, q_rank, kv_off, rank,
               rot, wq, wkv, eps, inv_freq, positions, slots, static_cast<float*>(cq), static_cast<float*>(k_cache));
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((latent_prep_kernel<__nv_bfloat16>), tokens, 256, 0, s, static_cast<const __nv_bfloat16*>(proj), stride, q_off,
               q_rank, kv_off, rank, rot, wq, wkv, eps, inv_freq, positions, slots, static_cast<__nv_bfloat16*>(cq),
               static_cast<__nv_bfloat16*>(k_cache));
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("latent_prep");
}

TIE_API int tie_latent_query_rot(int dtype, const void* q, long long q_stride, int dim, int rot, const float* inv_freq,
                                 const int* positions, void* folded, long long folded_stride, int rank, int heads, int tokens,
                                 cudaStream_t s) {
  TIE_REQUIRE(dim >= 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && heads > 0, "latent_query_rot: bad sizes dim=%d rank=%d rot=%d", dim, rank, rot);
  const long long items = static_cast<long long>(tokens) * heads;
  if (items <= 0 || rot == 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((latent_query_rot_kernel<float>), ceil_div(items, 4), 128, 0, s, static_cast<const float*>(q), q_stride, dim, rot,
               inv_freq, positions, static_cast<float*>(folded), folded_stride, rank, heads, items);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((latent_query_rot_kernel<__nv_bfloat16>), ceil_div(items, 4), 128, 0, s, static_cast<const __nv_bfloat16*>(q),
               q_stride, dim, rot, inv_freq, positions, static_cast<__nv_bfloat16*>(folded), folded_stride, rank, heads, items);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("latent_query_rot");
}

TIE_API int tie_head_gate_mul(int dtype, void* y, long long y_stride, const void* gate, long long gate_stride, int tokens,
                              int heads, int head_size, cudaStream_t s) {
  TIE_REQUIRE(heads > 0 && head_size > 0, "head_gate_mul: bad sizes heads=%d head_size=%d", heads, head_size);
  const long long total = static_cast<long long>(tokens) * heads * head_size;
  if (total <= 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((head_gate_mul_kernel<float>), ceil_div(total, 256), 256, 0, s, static_cast<float*>(y), y_stride,
               static_cast<const float*>(gate), gate_stride, heads * head_size, head_size, total);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((head_gate_mul_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, static_cast<__nv_bfloat16*>(y), y_stride,
               static_cast<const __nv_bfloat16*>(gate), gate_stride, heads * head_size, head_size, total);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("head_gate_mul");
}

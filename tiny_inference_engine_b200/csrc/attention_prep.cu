// What is done to the q, k and v of one token between their projection and attention, for attention layers
// that the per-head kernel (elementwise.cu) does not cover: biases, an RMS norm over the WHOLE q (and k)
// projection (all heads at once, `span` = heads * head size), a rotation of the first `rot` dimensions of each
// head, keys and values of different head sizes, and values blended with those of another layer:
//
//   q = proj_q + bq;  q = (q * inv(q over all heads)) * wq;  rotate;  written back in place
//   k likewise, into the key plane at the token's slot
//   v = proj_v + bv;  mode 1: v_first = v;  mode 2: v = (1 - lambda) v + lambda v_first;  into the value plane
//
// One block per token; sums, norms, angles and the blend in float. Planes: keys [pages, kv_heads, page, dim],
// values [pages, kv_heads, page, v_plane] with v_plane >= vdim (a model may keep its value heads padded with zeros
// to the key heads' size, so that kernels made for one head size serve it).
#include <math.h>

#include "common.cuh"

namespace tie {

struct PrepArgs {
  void* proj;                // [T, ...]: q at column q_off, k at k_off, v at v_off
  long long stride;
  int q_off, k_off, v_off;
  const float* bq;           // biases (null: none)
  const float* bk;
  const float* bv;
  const float* wq;           // norm weights over the whole projection (null: no norm)
  const float* wk;
  float eps;
  const float* inv_freq;     // [rot / 2] (null: no rotation)
  int rot;
  const int* positions;
  const int* slots;          // slot < 0: nothing is written to the planes
  void* k_cache;
  void* v_cache;             // null: this layer writes no keys and values
  int q_heads, kv_heads, dim, vdim, page_size;
  int v_plane;               // width of a row of the value plane (>= vdim; what lies beyond vdim is written as zero)
  int mix_mode;              // 0 none, 1 keep v as v_first, 2 blend with v_first
  float* v_first;            // [T, kv_heads * vdim]
  const float* lambda;       // device scalar
};

// buf[0, n) = proj + bias; then the norm over all n and the rotation, heads of `dim`.
template <typename T>
__device__ __forceinline__ void norm_rotate(float* buf, const T* src, const float* bias, const float* w, float eps, int n,
                                            int dim, int rot, const float* cs, float* scratch) {
  float ss = 0.0f;
  const bool wide = n % 4 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(bias) % 16 == 0;
  if (wide) {                                            // four elements a thread at a time
    for (int k = 4 * threadIdx.x; k < n; k += 4 * blockDim.x) {
      float v[4];
      load4(src + k, v);
      if (bias) {
        float b[4];
        load4(bias + k, b);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] += b[i];
      }
      store4(buf + k, v);
#pragma unroll
      for (int i = 0; i < 4; ++i) ss += v[i] * v[i];
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      float v = ld(src + i);
      if (bias) v += bias[i];
      buf[i] = v;
      ss += v * v;
    }
  }
  if (w) {
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(n) + eps);
    if (wide) {
      for (int k = 4 * threadIdx.x; k < n; k += 4 * blockDim.x)
#pragma unroll
        for (int i = 0; i < 4; ++i) buf[k + i] = (buf[k + i] * inv) * w[k + i];       // each thread its own elements
    } else {
      for (int i = threadIdx.x; i < n; i += blockDim.x) buf[i] = (buf[i] * inv) * w[i];
    }
  }
  __syncthreads();
  if (cs) {
    const int half = rot / 2, heads = n / dim;
    for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
      float* h = buf + (i / half) * dim;
      const int j = i % half;
      const float a = h[j], b = h[j + half], c = cs[j], sn = cs[half + j];
      h[j] = a * c - b * sn;
      h[j + half] = b * c + a * sn;
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256) qkv_span_prep_kernel(PrepArgs a) {
  pdl_sync();
  extern __shared__ float smem[];
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int nq = a.q_heads * a.dim, nk = a.kv_heads * a.dim, nv = a.kv_heads * a.vdim;
  float* cs = smem;                       // [rot]
  float* buf = smem + ((a.rot + 3) & ~3); // [max(nq, nk)], on a 16-byte boundary
  T* row = static_cast<T*>(a.proj) + static_cast<long long>(t) * a.stride;
  if (a.inv_freq) {
    const float p = static_cast<float>(a.positions[t]);
    for (int i = threadIdx.x; i < a.rot / 2; i += blockDim.x) {
      const float angle = p * a.inv_freq[i];
      cs[i] = cosf(angle);
      cs[a.rot / 2 + i] = sinf(angle);
    }
    __syncthreads();
  }
  const float* table = a.inv_freq ? cs : nullptr;
  norm_rotate<T>(buf, row + a.q_off, a.bq, a.wq, a.eps, nq, a.dim, a.rot, table, scratch);
  if (nq % 4 == 0 && reinterpret_cast<uintptr_t>(row + a.q_off) % 16 == 0) {
    for (int k = 4 * threadIdx.x; k < nq; k += 4 * blockDim.x) {
      float v[4];
      load4(buf + k, v);
      store4(row + a.q_off + k, v);
    }
  } else {
    for (int i = threadIdx.x; i < nq; i += blockDim.x) st(row + a.q_off + i, buf[i]);
  }
  if (a.v_cache == nullptr) return;
  __syncthreads();
  const int slot = a.slots[t];
  const long long page = slot >= 0 ? slot / a.page_size : 0;
  const int off = slot >= 0 ? slot % a.page_size : 0;
  norm_rotate<T>(buf, row + a.k_off, a.bk, a.wk, a.eps, nk, a.dim, a.rot, table, scratch);
  if (slot >= 0) {
    T* kc = static_cast<T*>(a.k_cache);
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
      const int g = i / a.dim, d = i % a.dim;
      st(kc + ((page * a.kv_heads + g) * a.page_size + off) * a.dim + d, buf[i]);
    }
  }
  const float lam = a.mix_mode == 2 ? *a.lambda : 0.0f;
  T* vc = static_cast<T*>(a.v_cache);
  for (int i = threadIdx.x; i < a.kv_heads * a.v_plane; i += blockDim.x) {
    const int g = i / a.v_plane, d = i % a.v_plane;
    float v = 0.0f;
    if (d < a.vdim) {
      const int j = g * a.vdim + d;
      v = ld(row + a.v_off + j);
      if (a.bv) v += a.bv[j];
      float* vf = a.v_first + static_cast<long long>(t) * nv + j;
      if (a.mix_mode == 1) *vf = v;
      else if (a.mix_mode == 2) v = (1.0f - lam) * v + lam * *vf;
    }
    if (slot >= 0) st(vc + ((page * a.kv_heads + g) * a.page_size + off) * a.v_plane + d, v);
  }
}

}  // namespace tie

using namespace tie;

TIE_API int tie_qkv_span_prep(int dtype, void* proj, long long stride, int q_off, int k_off, int v_off, const float* bq,
                              const float* bk, const float* bv, const float* wq, const float* wk, float eps,
                              const float* inv_freq, int rot, const int* positions, const int* slots, void* k_cache,
                              void* v_cache, int tokens, int q_heads, int kv_heads, int dim, int vdim, int v_plane,
                              int page_size, int mix_mode, float* v_first, const float* lambda, cudaStream_t s) {
  TIE_REQUIRE(v_plane >= vdim, "qkv_span_prep: rows of the value plane (%d) are narrower than a value head (%d)", v_plane, vdim);
  TIE_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && page_size > 0,
              "qkv_span_prep: bad sizes tokens=%d heads=%d/%d dim=%d vdim=%d page=%d", tokens, q_heads, kv_heads, dim, vdim,
              page_size);
  TIE_REQUIRE(inv_freq == nullptr || (rot > 0 && rot % 2 == 0 && rot <= dim), "qkv_span_prep: %d rotated dimensions of a head of %d",
              rot, dim);
  TIE_REQUIRE(mix_mode == 0 || (v_first != nullptr && (mix_mode == 1 || (mix_mode == 2 && lambda != nullptr))),
              "qkv_span_prep: value blending (mode %d) needs the first values and, to blend, its weight", mix_mode);
  if (tokens == 0) return kOk;
  if (inv_freq == nullptr) rot = 0;
  const PrepArgs a{proj, stride, q_off, k_off, v_off, bq, bk, bv, wq, wk, eps, inv_freq, rot, positions, slots, k_cache,
                   v_cache, q_heads, kv_heads, dim, vdim, page_size, v_plane, mix_mode, v_first, lambda};
  const int widest = q_heads * dim > kv_heads * dim ? q_heads * dim : kv_heads * dim;
  const size_t smem = static_cast<size_t>(((rot + 3) & ~3) + widest) * sizeof(float);
  TIE_REQUIRE(smem <= 200 * 1024, "qkv_span_prep: a projection of %d values does not fit shared memory", widest);
  if (dtype == TIE_F32) {
    auto kernel = qkv_span_prep_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    TIE_LAUNCH(kernel, tokens, 256, smem, s, a);
  } else if (dtype == TIE_BF16) {
    auto kernel = qkv_span_prep_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    TIE_LAUNCH(kernel, tokens, 256, smem, s, a);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("qkv_span_prep");
}

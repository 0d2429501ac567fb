// Small kernels around the residual stream and the gated units of layers with biases:
//
//   add_concat   x += delta (a tensor, or the partial sums of a split product added in order), then
//                out[t] = [x[t] | other[t]] in the storage type: the input of a product over the stream and a second
//                stream side by side (a model that mixes its embedding back in ahead of a span of layers).
//   glu_biased   out[t, i] = act(g[t, i] + bg[i]) * (u[t, i] + bu[i]), act the SiLU or the tanh form of GELU; out may be
//                wider than the unit: column I is then 1 and the columns after it 0, so that a product over
//                [W_down | bias | 0] adds the bias inside its float accumulator.
#include <math.h>

#include "common.cuh"

namespace tie {

template <typename T>
__global__ void __launch_bounds__(256) add_concat_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                         const float* __restrict__ part, long long part_stride, int splits,
                                                         const float* __restrict__ other, T* __restrict__ out, int dim) {
  pdl_sync();
  const long long t = blockIdx.x;
  float* xr = x + t * dim;
  for (int k = threadIdx.x; k < dim; k += blockDim.x) {
    float v = xr[k];
    if (delta != nullptr) {
      v += ld(delta + t * dim + k);
    } else if (part != nullptr) {
      float y = 0.0f;
      for (int z = 0; z < splits; ++z) y += part[z * part_stride + t * dim + k];
      v += y;
    }
    xr[k] = v;
    st(out + t * 2 * dim + k, v);
    st(out + t * 2 * dim + dim + k, other[t * dim + k]);
  }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void glu_biased_kernel(const T* __restrict__ gu, const float* __restrict__ bg, const float* __restrict__ bu,
                                  T* __restrict__ out, int inter, int out_width, int act, long long total) {
  pdl_sync();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / out_width;
  const int i = static_cast<int>(idx - t * out_width);
  if (i >= inter) {
    st(out + idx, i == inter ? 1.0f : 0.0f);
    return;
  }
  const float g = ld(gu + t * 2 * inter + i) + (bg ? bg[i] : 0.0f);
  const float u = ld(gu + t * 2 * inter + inter + i) + (bu ? bu[i] : 0.0f);
  const float a = act == 1 ? gelu_tanh_f(g) : g / (1.0f + expf(-g));
  st(out + idx, a * u);
}

// The same, 16 bytes a thread: `inter` and the output's width in whole vectors.
template <typename T>
__global__ void glu_biased_vec_kernel(const T* __restrict__ gu, const float* __restrict__ bg, const float* __restrict__ bu,
                                      T* __restrict__ out, int inter, int out_width, int act, long long total_vecs) {
  pdl_sync();
  constexpr int V = Vec16<T>::N;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total_vecs) return;
  const int per_row = out_width / V;
  const long long t = idx / per_row;
  const int i = static_cast<int>(idx - t * per_row) * V;
  Vec16<T> o;
  if (i >= inter) {
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = i + j == inter ? 1.0f : 0.0f;
  } else {
    Vec16<T> g, u;
    g.load(gu + t * 2 * inter + i);
    u.load(gu + t * 2 * inter + inter + i);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float gv = g.v[j] + (bg ? bg[i + j] : 0.0f), uv = u.v[j] + (bu ? bu[i + j] : 0.0f);
      o.v[j] = (act == 1 ? gelu_tanh_f(gv) : gv / (1.0f + expf(-gv))) * uv;
    }
  }
  o.store(out + t * out_width + i);
}

}  // namespace tie

using namespace tie;

TIE_API int tie_add_concat(int dtype, float* x, const void* delta, const float* part, long long part_stride, int splits,
                           const float* other, void* out, int tokens, int dim, cudaStream_t s) {
  TIE_REQUIRE(dim > 0 && tokens >= 0, "add_concat: bad sizes tokens=%d dim=%d", tokens, dim);
  if (tokens == 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((add_concat_kernel<float>), tokens, 256, 0, s, x, static_cast<const float*>(delta), part, part_stride, splits, other,
               static_cast<float*>(out), dim);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((add_concat_kernel<__nv_bfloat16>), tokens, 256, 0, s, x, static_cast<const __nv_bfloat16*>(delta), part, part_stride,
               splits, other, static_cast<__nv_bfloat16*>(out), dim);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("add_concat");
}

TIE_API int tie_glu_biased(int dtype, const void* gu, const float* bg, const float* bu, void* out, int tokens, int inter,
                           int out_width, int act, cudaStream_t s) {
  TIE_REQUIRE(inter > 0 && out_width >= inter && (act == 0 || act == 1), "glu_biased: bad sizes inter=%d out width=%d act=%d", inter,
              out_width, act);
  const long long total = static_cast<long long>(tokens) * out_width;
  if (total <= 0) return kOk;
  const int v = dtype == TIE_BF16 ? 8 : 4;
  if ((dtype == TIE_BF16 || dtype == TIE_F32) && inter % v == 0 && out_width % v == 0 && reinterpret_cast<uintptr_t>(gu) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    const long long vecs = total / v;
    if (dtype == TIE_F32) {
      TIE_LAUNCH((glu_biased_vec_kernel<float>), ceil_div(vecs, 256), 256, 0, s, static_cast<const float*>(gu), bg, bu,
                 static_cast<float*>(out), inter, out_width, act, vecs);
    } else {
      TIE_LAUNCH((glu_biased_vec_kernel<__nv_bfloat16>), ceil_div(vecs, 256), 256, 0, s, static_cast<const __nv_bfloat16*>(gu), bg, bu,
                 static_cast<__nv_bfloat16*>(out), inter, out_width, act, vecs);
    }
    TIE_RETURN_LAUNCH("glu_biased");
  }
  if (dtype == TIE_F32) {
    TIE_LAUNCH((glu_biased_kernel<float>), ceil_div(total, 256), 256, 0, s, static_cast<const float*>(gu), bg, bu,
               static_cast<float*>(out), inter, out_width, act, total);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((glu_biased_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, static_cast<const __nv_bfloat16*>(gu), bg, bu,
               static_cast<__nv_bfloat16*>(out), inter, out_width, act, total);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("glu_biased");
}

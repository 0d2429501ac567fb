// What stands around the recurrence S <- diag(decay) S + k u^T, o = S^T q (delta_rule.cu in its plain mode) for two
// mixers that have no delta correction:
//
//   gated linear attention   q, k, v straight from their projections (q scaled), a decay per head and key channel,
//                            decay = sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau), z the decay projection plus its bias;
//                            read-out: o / rms(o) * w * act(gate) per head.
//   state-space duality      x, B and C behind a short causal convolution with bias and SiLU; a step size per head,
//                            dt = softplus(raw + bias); decay = exp(-exp(A_log) dt) for the whole head; the write is
//                            dt * B x^T; read-out: (o + D x) * silu(z), normed in equal parts of the row, times w.
//
// Kernels (float inside; T is the storage type of the projections and of the outputs that feed a product):
//   gla_prep      one block per token.
//   ssd_prep      one block per (token, unit): units are the heads of C, of B and of x, and one for the step sizes.
//                 The convolution's first taps - 1 inputs come from the rows ahead in the step or from the tail that
//                 the sequence's state slot keeps behind S (channels in the order C, B, x).
//   head_norm_gate  one warp per (token, head).
//   ssd_out       one block per (token, part of the row).
#include <math.h>

#include "common.cuh"

namespace tie {

__device__ __forceinline__ float lr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float lr_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename T>
__global__ void __launch_bounds__(256) gla_prep_kernel(const T* __restrict__ proj, long long stride, int q_off, int k_off,
                                                       int v_off, int nqk, int nv, float q_scale, float inv_tau,
                                                       const float* __restrict__ z_bias, float* __restrict__ qn,
                                                       float* __restrict__ kn, float* __restrict__ vn,
                                                       float* __restrict__ decay, long long decay_stride) {
  pdl_sync();
  const long long t = blockIdx.x;
  const T* row = proj + t * stride;
  for (int c = threadIdx.x; c < nqk; c += blockDim.x) {
    qn[t * nqk + c] = ld(row + q_off + c) * q_scale;
    kn[t * nqk + c] = ld(row + k_off + c);
    float* a = decay + t * decay_stride + c;
    const float z = *a + (z_bias ? z_bias[c] : 0.0f);
    *a = expf(-lr_softplus(-z) * inv_tau);
  }
  for (int c = threadIdx.x; c < nv; c += blockDim.x) vn[t * nv + c] = ld(row + v_off + c);
}

struct SsdShape {
  int heads, groups, state, vdim, taps;
};

template <typename T>
__global__ void __launch_bounds__(128) ssd_prep_kernel(const T* __restrict__ proj, long long stride, int c_off, int b_off,
                                                       int x_off, int dt_off, const float* __restrict__ conv_w,
                                                       const float* __restrict__ conv_b, const float* __restrict__ state,
                                                       long long state_stride, long long conv_state_off,
                                                       const int* __restrict__ seq_of_row,
                                                       const int* __restrict__ query_start,
                                                       const int* __restrict__ state_slots, SsdShape sh,
                                                       const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                       float* __restrict__ cn, float* __restrict__ bn,
                                                       float* __restrict__ xn, float* __restrict__ dt,
                                                       float* __restrict__ decay) {
  pdl_sync();
  const int t = blockIdx.x, unit = blockIdx.y;
  const int G = sh.groups, H = sh.heads, N = sh.state, vdim = sh.vdim, taps = sh.taps;
  const int ngn = G * N, nv = H * vdim, C = 2 * ngn + nv;
  const T* row = proj + static_cast<long long>(t) * stride;
  if (unit == 2 * G + H) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float step = lr_softplus(ld(row + dt_off + h) + dt_bias[h]);
      dt[static_cast<long long>(t) * H + h] = step;
      decay[static_cast<long long>(t) * H + h] = expf(-expf(a_log[h]) * step);
    }
    return;
  }
  const int s = seq_of_row[t];
  const int j = t - query_start[s];          // tokens of this sequence ahead of this one in the step
  const int slot = state_slots[s];
  const float* tail = slot >= 0 ? state + slot * state_stride + conv_state_off : nullptr;
  const bool is_x = unit >= 2 * G;
  const int width = is_x ? vdim : N;
  const int c0 = is_x ? 2 * ngn + (unit - 2 * G) * vdim : unit * N;      // the unit's first channel of all C
  float* dst = is_x ? xn + static_cast<long long>(t) * nv + (unit - 2 * G) * vdim
                    : (unit < G ? cn + static_cast<long long>(t) * ngn + unit * N
                                : bn + static_cast<long long>(t) * ngn + (unit - G) * N);
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const int c = c0 + d;
    const int col = c < ngn ? c_off + c : (c < 2 * ngn ? b_off + (c - ngn) : x_off + (c - 2 * ngn));
    float y = conv_b ? conv_b[c] : 0.0f;
    for (int i = 0; i < taps; ++i) {
      const int back = taps - 1 - i;         // this tap's input is `back` tokens ahead of the current one
      float in;
      if (back <= j) in = ld(row - static_cast<long long>(back) * stride + col);
      else in = tail ? tail[static_cast<long long>(j + i) * C + c] : 0.0f;
      y = fmaf(conv_w[c * taps + i], in, y);
    }
    dst[d] = y * lr_sigmoid(y);
  }
}

// out[t, h] = (o[t, h] / rms(o[t, h])) * w * act(gate[t, h]); act 0: sigmoid, 1: silu. The gate has the storage type.
template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate,
                                                             long long gate_stride, const float* __restrict__ w, float eps,
                                                             T* __restrict__ out, int heads, int vdim, int act,
                                                             long long items) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / heads;
  const int h = static_cast<int>(item % heads);
  const float* x = o + item * vdim;
  float ss = 0.0f;
  for (int d = lane; d < vdim; d += 32) ss += x[d] * x[d];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(vdim) + eps);
  for (int d = lane; d < vdim; d += 32) {
    const float g = ld(gate + t * gate_stride + h * vdim + d);
    const float a = act == 1 ? g * lr_sigmoid(g) : lr_sigmoid(g);
    st(out + item * vdim + d, ((x[d] * inv) * w[d]) * a);
  }
}

// y = (o + skip[h] x) * silu(z), each of `parts` equal parts of the row divided by its own root mean square, times w.
template <typename T>
__global__ void __launch_bounds__(256) ssd_out_kernel(const float* __restrict__ o, const float* __restrict__ xn,
                                                      const T* __restrict__ z, long long z_stride,
                                                      const float* __restrict__ skip, const float* __restrict__ w, float eps,
                                                      T* __restrict__ out, int inner, int vdim, int parts) {
  pdl_sync();
  __shared__ float scratch[33];
  const long long t = blockIdx.x;
  const int part = blockIdx.y, size = inner / parts, c0 = part * size;
  float ss = 0.0f;
  for (int d = threadIdx.x; d < size; d += blockDim.x) {
    const int c = c0 + d;
    const float g = ld(z + t * z_stride + c);
    const float y = fmaf(skip[c / vdim], xn[t * inner + c], o[t * inner + c]) * (g * lr_sigmoid(g));
    ss += y * y;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(size) + eps);
  for (int d = threadIdx.x; d < size; d += blockDim.x) {
    const int c = c0 + d;
    const float g = ld(z + t * z_stride + c);
    const float y = fmaf(skip[c / vdim], xn[t * inner + c], o[t * inner + c]) * (g * lr_sigmoid(g));
    st(out + t * inner + c, (y * inv) * w[c]);
  }
}

}  // namespace tie

using namespace tie;

#define TIE_BY_DTYPE(dtype, CALL)                        \
  do {                                                   \
    if (dtype == TIE_F32) {                              \
      using T = float;                                   \
      CALL;                                              \
    } else if (dtype == TIE_BF16) {                      \
      using T = __nv_bfloat16;                           \
      CALL;                                              \
    } else {                                             \
      set_error("unknown dtype code %d", dtype);         \
      return kBadArgument;                               \
    }                                                    \
  } while (0)

TIE_API int tie_gla_prep(int dtype, const void* proj, long long stride, int q_off, int k_off, int v_off, int tokens, int heads,
                         int dim, int vdim, float q_scale, float tau, const float* z_bias, float* qn, float* kn, float* vn,
                         float* decay, long long decay_stride, cudaStream_t s) {
  TIE_REQUIRE(heads > 0 && dim > 0 && vdim > 0 && tau > 0.0f, "gla_prep: bad sizes heads=%d dim=%d vdim=%d tau=%g", heads, dim,
              vdim, static_cast<double>(tau));
  if (tokens <= 0) return kOk;
  TIE_BY_DTYPE(dtype, TIE_LAUNCH((gla_prep_kernel<T>), tokens, 256, 0, s, static_cast<const T*>(proj), stride, q_off, k_off, v_off,
                                 heads * dim, heads * vdim, q_scale, 1.0f / tau, z_bias, qn, kn, vn, decay, decay_stride));
  TIE_RETURN_LAUNCH("gla_prep");
}

TIE_API int tie_ssd_prep(int dtype, const void* proj, long long stride, int c_off, int b_off, int x_off, int dt_off,
                         const float* conv_w, const float* conv_b, const float* state, long long state_stride,
                         long long conv_state_off, const int* seq_of_row, const int* query_start, const int* state_slots,
                         int tokens, int heads, int groups, int state_size, int vdim, int taps, const float* dt_bias,
                         const float* a_log, float* cn, float* bn, float* xn, float* dt, float* decay, cudaStream_t s) {
  TIE_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && state_size > 0 && vdim > 0 && taps >= 1 && taps <= 16,
              "ssd_prep: bad shape heads=%d groups=%d state=%d vdim=%d taps=%d (1 to 16)", heads, groups, state_size, vdim, taps);
  if (tokens <= 0) return kOk;
  const int units = 2 * groups + heads + 1;
  TIE_REQUIRE(units <= 65535, "ssd_prep: %d heads exceed the grid", heads);
  const SsdShape sh{heads, groups, state_size, vdim, taps};
  TIE_BY_DTYPE(dtype, TIE_LAUNCH((ssd_prep_kernel<T>), dim3(tokens, units), 128, 0, s, static_cast<const T*>(proj), stride, c_off,
                                 b_off, x_off, dt_off, conv_w, conv_b, state, state_stride, conv_state_off, seq_of_row,
                                 query_start, state_slots, sh, dt_bias, a_log, cn, bn, xn, dt, decay));
  TIE_RETURN_LAUNCH("ssd_prep");
}

TIE_API int tie_head_norm_gate(int dtype, const float* o, const void* gate, long long gate_stride, const float* w, float eps,
                               void* out, int tokens, int heads, int vdim, int act, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0 && (act == 0 || act == 1), "head_norm_gate: bad sizes tokens=%d heads=%d vdim=%d act=%d",
              tokens, heads, vdim, act);
  const long long items = static_cast<long long>(tokens) * heads;
  if (items == 0) return kOk;
  TIE_BY_DTYPE(dtype, TIE_LAUNCH((head_norm_gate_kernel<T>), ceil_div(items, 4), 128, 0, s, o, static_cast<const T*>(gate),
                                 gate_stride, w, eps, static_cast<T*>(out), heads, vdim, act, items));
  TIE_RETURN_LAUNCH("head_norm_gate");
}

TIE_API int tie_ssd_out(int dtype, const float* o, const float* xn, const void* z, long long z_stride, const float* skip,
                        const float* w, float eps, void* out, int tokens, int heads, int vdim, int parts, cudaStream_t s) {
  TIE_REQUIRE(heads > 0 && vdim > 0 && parts > 0 && (heads * vdim) % parts == 0 && parts <= 65535,
              "ssd_out: %d heads of %d do not split into %d equal parts", heads, vdim, parts);
  if (tokens <= 0) return kOk;
  TIE_BY_DTYPE(dtype, TIE_LAUNCH((ssd_out_kernel<T>), dim3(tokens, parts), 256, 0, s, o, xn, static_cast<const T*>(z), z_stride,
                                 skip, w, eps, static_cast<T*>(out), heads * vdim, vdim, parts));
  TIE_RETURN_LAUNCH("ssd_out");
}

// A product per head: out[t, h, :N] = w[h] a[t, h, :K] for every head h at once, bfloat16 on the tensor cores
// (mma.sync m16n8k16, float accumulation). The heads' inputs lie side by side in a row of `a` (head h at column
// h * a_head) and so do their outputs (at h * o_head); w is [heads, N, K]. This is what stands on either side of
// attention over one latent per token: the per-head map from the query to the latent's space, and from the weighted
// sum of latents to the head's value.
//
// One CTA per (128 tokens, 64 output columns, head): eight warps as 4 x 2, each 32 x 32 of the tile; operands come
// through two shared-memory buffers filled by cp.async, k in steps of 32, rows padded to five 16-byte pieces so that
// ldmatrix meets no bank twice. Few tokens (decode) stay with the CUDA-core kernel that streams the weights once.
#include "attention_mma.cuh"

namespace tie {

constexpr int kHgM = 128, kHgN = 64, kHgK = 32, kHgThreads = 256, kHgStride = 5;     // pieces of 16 bytes from row to row

__global__ void __launch_bounds__(kHgThreads) gemm_heads_mma_kernel(const __nv_bfloat16* __restrict__ a, long long lda, int a_head,
                                                                    const __nv_bfloat16* __restrict__ w,
                                                                    __nv_bfloat16* __restrict__ out, long long ldo, int o_head,
                                                                    int M, int N, int K) {
  pdl_sync();
  __shared__ __align__(16) unsigned char smem[2 * (kHgM + kHgN) * kHgStride * 16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp >> 1, wn = warp & 1;
  const int m0 = blockIdx.y * kHgM, n0 = blockIdx.x * kHgN, h = blockIdx.z;
  const __nv_bfloat16* ah = a + static_cast<long long>(h) * a_head;
  const __nv_bfloat16* wh = w + static_cast<long long>(h) * N * K;
  const uint32_t base = smem_addr(smem);
  constexpr uint32_t kBuf = (kHgM + kHgN) * kHgStride * 16, kWOff = kHgM * kHgStride * 16;
  auto at = [](int row, int chunk) { return static_cast<uint32_t>((row * kHgStride + chunk) << 4); };
  auto fetch = [&](int k0, uint32_t dst) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {                 // 128 rows x 4 pieces of the token tile
      const int idx = threadIdx.x + i * kHgThreads;
      const int r = idx >> 2, c = idx & 3;
      const bool valid = m0 + r < M && k0 + c * 8 < K;
      cp_async16(dst + at(r, c), valid ? ah + static_cast<long long>(m0 + r) * lda + k0 + c * 8 : ah, valid ? 16 : 0);
    }
    {                                             // 64 rows x 4 pieces of the weight tile
      const int r = threadIdx.x >> 2, c = threadIdx.x & 3;
      const bool valid = n0 + r < N && k0 + c * 8 < K;
      cp_async16(dst + kWOff + at(r, c), valid ? wh + static_cast<long long>(n0 + r) * K + k0 + c * 8 : wh, valid ? 16 : 0);
    }
  };
  float acc[2][4][4] = {};
  const int steps = (K + kHgK - 1) / kHgK;
  fetch(0, base);
  cp_async_commit();
  for (int s = 0; s < steps; ++s) {
    const uint32_t buf = base + (s & 1) * kBuf;
    cp_async_wait<0>();
    __syncthreads();
    if (s + 1 < steps) fetch((s + 1) * kHgK, base + ((s + 1) & 1) * kBuf);
    cp_async_commit();
#pragma unroll
    for (int ks = 0; ks < kHgK / 16; ++ks) {
      uint32_t af[2][4], bf[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) ldmatrix_x4(af[mt], buf + at(wm * 32 + mt * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
      for (int np = 0; np < 2; ++np)
        ldmatrix_x4(bf[np], buf + kWOff + at(wn * 32 + np * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          mma_bf16(acc[mt][2 * np], af[mt], bf[np][0], bf[np][1]);
          mma_bf16(acc[mt][2 * np + 1], af[mt], bf[np][2], bf[np][3]);
        }
    }
  }
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int t = m0 + wm * 32 + mt * 16 + g + 8 * half;
      if (t >= M) continue;
      __nv_bfloat16* dst = out + static_cast<long long>(t) * ldo + static_cast<long long>(h) * o_head;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int n = n0 + wn * 32 + nt * 8 + 2 * tq;
        if (n < N) *reinterpret_cast<uint32_t*>(dst + n) = pack_bf16(acc[mt][nt][2 * half], acc[mt][nt][2 * half + 1]);
      }
    }
}

}  // namespace tie

using namespace tie;

// Whether the tensor-core kernel takes these sizes and addresses (else the CUDA-core kernel does).
TIE_API int tie_gemm_heads_mma_takes(const void* a, long long lda, int a_head, const void* w, const void* out, long long ldo,
                                     int o_head, int N, int K) {
  return K % 8 == 0 && N % 2 == 0 && lda % 8 == 0 && a_head % 8 == 0 && ldo % 2 == 0 && o_head % 2 == 0 &&
         reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0;
}

TIE_API int tie_gemm_heads_mma(const void* a, long long lda, int a_head, const void* w, void* out, long long ldo, int o_head,
                               int M, int N, int K, int heads, cudaStream_t s) {
  TIE_REQUIRE(M >= 0 && N > 0 && K > 0 && heads > 0 && heads <= 65535, "gemm_heads: bad sizes M=%d N=%d K=%d heads=%d", M, N, K, heads);
  TIE_REQUIRE(tie_gemm_heads_mma_takes(a, lda, a_head, w, out, ldo, o_head, N, K),
              "gemm_heads on the tensor cores: K=%d and the heads' offsets must be whole 16-byte vectors, N=%d even", K, N);
  if (M == 0) return kOk;
  TIE_LAUNCH(gemm_heads_mma_kernel, dim3(ceil_div(N, kHgN), ceil_div(M, kHgM), heads), kHgThreads, 0, s,
             static_cast<const __nv_bfloat16*>(a), lda, a_head, static_cast<const __nv_bfloat16*>(w),
             static_cast<__nv_bfloat16*>(out), ldo, o_head, M, N, K);
  TIE_RETURN_LAUNCH("gemm_heads_mma");
}

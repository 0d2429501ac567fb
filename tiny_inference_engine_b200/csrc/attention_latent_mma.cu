// Attention over one cached row per token for all heads (attention_latent.cu says why), bfloat16 on the tensor cores.
//
// Every head's query has `kd` dimensions (a folded latent part and a rotated part) and reads the same keys, rows of kd
// in one plane; a key's first `rank` elements are its value. So the rows of an MMA tile are (token, head) pairs that
// share each key tile: a CTA takes 32 of them (32 / heads tokens, or 32 heads of one token), eight warps as two row
// groups of 16 times four column groups. Per tile of 64 keys (cp.async into two buffers in turn, rows padded to an
// odd number of 16-byte pieces so that ldmatrix meets no bank twice):
//   1. scores: column group c takes keys [16c, 16c + 16): S = Q K^T over kd with mma.sync m16n8k16, float, to shared memory;
//   2. every warp reads its 16 rows of S, masks (causal, window), updates the running maximum and sum (float; the four
//      warps of a row group compute the same numbers) and turns the weights into bfloat16 A fragments;
//   3. values: column group c owns every fourth block of 16 value columns: acc += P V with V read transposed from
//      the same key tile; the float weights enter as two bfloat16 terms, hi + lo, each with an MMA of its own.
// Prompt rows write acc / sum; rows of sequences that bring one token split their keys over CTAs and leave
// (acc, max, sum) per split in the layout that `tie_attention_merge` adds up.
#include "attention_mma.cuh"

namespace tie {

constexpr int kLatRows = 32;
constexpr int kLatKeys = 64;
constexpr int kLatThreads = 256;

struct LatentArgs {
  const __nv_bfloat16* q;          // [T, heads * kd], rows q_stride apart
  const __nv_bfloat16* keys;       // [pages, 1, page_size, kd]
  __nv_bfloat16* out;              // [T, heads * rank]
  const int* query_start;          // [S + 1]
  const int* context_lens;         // [S]
  const int* block_tables;         // [S, max_blocks]
  long long q_stride;
  int max_blocks, heads, kd, rank, page_size, window;
  float scale_log2;                // scale * log2(e)
  // sequences that bring one token, their keys cut into splits
  const int* seq_list;
  int n_list, split_keys, max_splits;
  float* scratch;                  // [n_list, heads, max_splits, rank + 2]
};

__device__ __forceinline__ uint32_t lat_at(int row, int chunk, int stride_chunks) { return static_cast<uint32_t>((row * stride_chunks + chunk) << 4); }

// MAXP: blocks of 16 value columns a warp may own (rank <= 64 * MAXP). SPLIT: the one-token mode.
template <int MAXP, bool SPLIT>
__global__ void __launch_bounds__(kLatThreads) latent_attention_mma_kernel(LatentArgs a) {
  pdl_sync();
  extern __shared__ __align__(16) unsigned char lat_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rg = warp >> 2, cg = warp & 3;                 // row group, column group
  const int g = lane >> 2, tq = lane & 3;
  const int H = a.heads, kd = a.kd, rank = a.rank;
  const int hc = H < kLatRows ? H : kLatRows;              // heads of a CTA
  const int bq = SPLIT ? 1 : kLatRows / hc;                // tokens of a CTA
  const int h0 = blockIdx.z * hc;
  int s, t0, n_tok, pos0, key_lo, key_hi, split = 0, li = 0;
  if (SPLIT) {
    li = blockIdx.y;
    split = blockIdx.x;
    s = a.seq_list[li];
    t0 = a.query_start[s];
    n_tok = 1;
    pos0 = a.context_lens[s] - 1;
    if (pos0 < 0) return;
    const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    key_lo = lo0 + split * a.split_keys;
    if (key_lo > pos0) return;
    key_hi = split == a.max_splits - 1 ? pos0 : min(pos0, key_lo + a.split_keys - 1);
  } else {
    s = blockIdx.y;
    const int qs0 = a.query_start[s], nq = a.query_start[s + 1] - qs0;
    const int first = blockIdx.x * bq;
    if (first >= nq) return;
    t0 = qs0 + first;
    n_tok = min(bq, nq - first);
    pos0 = a.context_lens[s] - nq + first;                 // position of the CTA's first token
    key_lo = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    key_hi = pos0 + n_tok - 1;
  }
  const int ch = kd >> 3;                                  // 16-byte pieces of a row
  const int sc = ch | 1;                                   // pieces from one row to the next in shared memory
  const uint32_t q_tile = smem_addr(lat_smem);
  const uint32_t k_tile0 = q_tile + kLatRows * sc * 16;
  const uint32_t k_bytes = kLatKeys * sc * 16;
  float* sbuf = reinterpret_cast<float*>(lat_smem + kLatRows * sc * 16 + 2 * k_bytes);      // [32][kLatKeys + 4]
  constexpr int kSLd = kLatKeys + 4;
  const int* table = a.block_tables + static_cast<long long>(s) * a.max_blocks;

  // queries: row r = (token r / hc, head h0 + r % hc)
  for (int i = threadIdx.x; i < kLatRows * ch; i += kLatThreads) {
    const int r = i / ch, c = i - r * ch;
    const int tok = r / hc, head = h0 + r % hc;
    const bool valid = tok < n_tok && head < H;
    const __nv_bfloat16* src = valid ? a.q + static_cast<long long>(t0 + tok) * a.q_stride + static_cast<long long>(head) * kd + c * 8 : a.q;
    cp_async16(q_tile + lat_at(r, c, sc), src, valid ? 16 : 0);
  }
  // Where each key of a tile lives (element offset of its row in the plane, or -1 outside the CTA's range) is worked
  // out by 64 threads a tile ahead of the copy that uses it, so that the copy loop has no division and no load that
  // an address depends on: warp w copies keys w, w + 8, ..., lane l the pieces l, l + 32, ...
  long long* row_off = reinterpret_cast<long long*>(sbuf + kLatRows * kSLd);         // [2][kLatKeys]
  auto locate = [&](int tile) {
    if (threadIdx.x < kLatKeys) {
      const int key = tile * kLatKeys + threadIdx.x;
      long long off = -1;
      if (key >= key_lo && key <= key_hi) off = (static_cast<long long>(table[key / a.page_size]) * a.page_size + key % a.page_size) * kd;
      row_off[(tile & 1) * kLatKeys + threadIdx.x] = off;
    }
  };
  auto fetch = [&](int tile, uint32_t dst) {
    const long long* off = row_off + (tile & 1) * kLatKeys;
    for (int r = warp; r < kLatKeys; r += kLatThreads / 32) {
      const long long o = off[r];
      const __nv_bfloat16* src = o >= 0 ? a.keys + o : a.keys;
      for (int c = lane; c < ch; c += 32) cp_async16(dst + lat_at(r, c, sc), src + (o >= 0 ? c * 8 : 0), o >= 0 ? 16 : 0);
    }
  };
  const int first_tile = key_lo / kLatKeys, last_tile = key_hi / kLatKeys;
  locate(first_tile);
  locate(first_tile + 1);
  __syncthreads();
  fetch(first_tile, k_tile0);
  cp_async_commit();

  // this thread's two rows: g and g + 8 of its row group
  int pos_r[2], lo_r[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = rg * 16 + g + 8 * half;
    const int tok = r / hc;
    const bool valid = tok < n_tok && h0 + r % hc < H;
    pos_r[half] = valid ? pos0 + tok : -1;                                   // no key for a row that is not there
    lo_r[half] = a.window > 0 ? max(0, pos_r[half] - a.window + 1) : 0;
    if (SPLIT) lo_r[half] = max(lo_r[half], key_lo);
    if (SPLIT && valid) pos_r[half] = key_hi;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float acc[MAXP][2][4];
#pragma unroll
  for (int p = 0; p < MAXP; ++p)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[p][e >> 2][e & 3] = 0.0f;
  const int pairs = rank >> 4;                             // blocks of 16 value columns

  for (int tile = first_tile; tile <= last_tile; ++tile) {
    const uint32_t k_tile = k_tile0 + ((tile - first_tile) & 1) * k_bytes;
    cp_async_wait<0>();
    __syncthreads();                                       // this tile is there; everyone is through with the other buffer and with S
    if (tile < last_tile) fetch(tile + 1, k_tile0 + ((tile + 1 - first_tile) & 1) * k_bytes);
    cp_async_commit();
    locate(tile + 2);                                      // read by the copy that the next round issues, behind its barrier
    // 1. scores of keys [16 cg, 16 cg + 16) for this row group
    float sc4[2][4] = {}, sc4b[2][4] = {};                 // two sets of sums in turn: twice as many MMAs in flight
    const uint32_t q_row = q_tile + lat_at(rg * 16 + (lane & 15), lane >> 4, sc);
    const uint32_t k_row = k_tile + lat_at(cg * 16 + (lane & 7) + ((lane >> 4) << 3), (lane >> 3) & 1, sc);
    const int ksteps = kd >> 4;
    int ks = 0;
    for (; ks + 1 < ksteps; ks += 2) {
      uint32_t qa[4], kb[4], qa2[4], kb2[4];
      ldmatrix_x4(qa, q_row + (ks << 5));
      ldmatrix_x4(kb, k_row + (ks << 5));
      ldmatrix_x4(qa2, q_row + ((ks + 1) << 5));
      ldmatrix_x4(kb2, k_row + ((ks + 1) << 5));
      mma_bf16(sc4[0], qa, kb[0], kb[1]);
      mma_bf16(sc4[1], qa, kb[2], kb[3]);
      mma_bf16(sc4b[0], qa2, kb2[0], kb2[1]);
      mma_bf16(sc4b[1], qa2, kb2[2], kb2[3]);
    }
    if (ks < ksteps) {
      uint32_t qa[4], kb[4];
      ldmatrix_x4(qa, q_row + (ks << 5));
      ldmatrix_x4(kb, k_row + (ks << 5));
      mma_bf16(sc4[0], qa, kb[0], kb[1]);
      mma_bf16(sc4[1], qa, kb[2], kb[3]);
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc4[nt][e] += sc4b[nt][e];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float* dst = sbuf + (rg * 16 + g) * kSLd + cg * 16 + nt * 8 + 2 * tq;
      dst[0] = sc4[nt][0], dst[1] = sc4[nt][1];
      dst[8 * kSLd] = sc4[nt][2], dst[8 * kSLd + 1] = sc4[nt][3];
    }
    __syncthreads();
    // 2. this warp's 16 rows over the tile's 64 keys, in the layout of eight accumulator tiles
    float p[8][4];
    const int key0 = tile * kLatKeys;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float2 v = *reinterpret_cast<const float2*>(sbuf + (rg * 16 + g + 8 * half) * kSLd + j * 8 + 2 * tq);
        const int key = key0 + j * 8 + 2 * tq;
        p[j][2 * half] = key >= lo_r[half] && key <= pos_r[half] ? v.x * a.scale_log2 : -INFINITY;
        p[j][2 * half + 1] = key + 1 >= lo_r[half] && key + 1 <= pos_r[half] ? v.y * a.scale_log2 : -INFINITY;
      }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fmaxf(p[j][2 * half], p[j][2 * half + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[half], mx);
      const float base = m_new == -INFINITY ? 0.0f : m_new;       // a row with no key yet: everything stays zero
      const float corr = exp2f(m[half] - base);
      float sum = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        p[j][2 * half] = exp2f(p[j][2 * half] - base);
        p[j][2 * half + 1] = exp2f(p[j][2 * half + 1] - base);
        sum += p[j][2 * half] + p[j][2 * half + 1];
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[half] = l[half] * corr + sum;
      m[half] = m_new;
#pragma unroll
      for (int q = 0; q < MAXP; ++q)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) acc[q][nt][2 * half] *= corr, acc[q][nt][2 * half + 1] *= corr;
    }
    // 3. values: blocks cg, cg + 4, ... of 16 columns
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {                       // 16 keys per MMA k-step
      uint32_t pa[4];
      pa[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
      pa[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
      pa[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
      pa[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
      // the float weights enter the product as two bfloat16 terms, hi + lo: 16 bits of mantissa instead of 8
      uint32_t pr[4];
      pr[0] = pack_bf16_rest(p[2 * kk][0], p[2 * kk][1], pa[0]);
      pr[1] = pack_bf16_rest(p[2 * kk][2], p[2 * kk][3], pa[1]);
      pr[2] = pack_bf16_rest(p[2 * kk + 1][0], p[2 * kk + 1][1], pa[2]);
      pr[3] = pack_bf16_rest(p[2 * kk + 1][2], p[2 * kk + 1][3], pa[3]);
#pragma unroll
      for (int q = 0; q < MAXP; ++q) {
        const int blk = cg + 4 * q;
        if (blk < pairs) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, k_tile + lat_at(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), blk * 2 + (lane >> 4), sc));
          mma_bf16(acc[q][0], pa, vb[0], vb[1]);
          mma_bf16(acc[q][1], pa, vb[2], vb[3]);
          mma_bf16(acc[q][0], pr, vb[0], vb[1]);
          mma_bf16(acc[q][1], pr, vb[2], vb[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  // results: rows g and g + 8, columns blk * 16 + nt * 8 + 2 tq
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = rg * 16 + g + 8 * half;
    const int tok = r / hc, head = h0 + r % hc;
    if (tok >= n_tok || head >= H) continue;
    if (SPLIT) {
      float* dst = a.scratch + ((static_cast<long long>(li) * H + head) * a.max_splits + split) * (rank + 2);
#pragma unroll
      for (int q = 0; q < MAXP; ++q) {
        const int blk = cg + 4 * q;
        if (blk >= pairs) continue;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          dst[blk * 16 + nt * 8 + 2 * tq] = acc[q][nt][2 * half];
          dst[blk * 16 + nt * 8 + 2 * tq + 1] = acc[q][nt][2 * half + 1];
        }
      }
      if (cg == 0 && tq == 0) {
        // the merge works with natural exponents: max in units of the score, sums relative to it
        dst[rank] = m[half] * 0.6931471805599453f;
        dst[rank + 1] = l[half];
      }
    } else {
      const float inv = l[half] > 0.0f ? 1.0f / l[half] : 0.0f;
      __nv_bfloat16* dst = a.out + (static_cast<long long>(t0 + tok) * H + head) * rank;
#pragma unroll
      for (int q = 0; q < MAXP; ++q) {
        const int blk = cg + 4 * q;
        if (blk >= pairs) continue;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
          *reinterpret_cast<uint32_t*>(dst + blk * 16 + nt * 8 + 2 * tq) = pack_bf16(acc[q][nt][2 * half] * inv, acc[q][nt][2 * half + 1] * inv);
      }
    }
  }
}

static size_t latent_smem(int kd) {
  const int sc = (kd / 8) | 1;
  return static_cast<size_t>(kLatRows + 2 * kLatKeys) * sc * 16 + static_cast<size_t>(kLatRows) * (kLatKeys + 4) * sizeof(float) +
         2 * kLatKeys * sizeof(long long);
}

template <bool SPLIT>
static int launch_latent(const LatentArgs& a, dim3 grid, cudaStream_t s) {
  const size_t smem = latent_smem(a.kd);
#define TIE_LATENT_CASE(P)                                                                                              \
  do {                                                                                                                  \
    static bool raised = false;                                                                                         \
    if (!raised) {                                                                                                      \
      cudaFuncSetAttribute(latent_attention_mma_kernel<P, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      raised = true;                                                                                                    \
    }                                                                                                                   \
    TIE_LAUNCH((latent_attention_mma_kernel<P, SPLIT>), grid, kLatThreads, smem, s, a);                                   \
  } while (0)
  if (a.rank <= 128) TIE_LATENT_CASE(2);
  else if (a.rank <= 256) TIE_LATENT_CASE(4);
  else TIE_LATENT_CASE(8);
#undef TIE_LATENT_CASE
  TIE_RETURN_LAUNCH("latent_attention_mma");
}

static int check_latent(const LatentArgs& a) {
  TIE_REQUIRE(a.heads > 0 && a.kd > 0 && a.kd % 16 == 0 && a.rank > 0 && a.rank % 16 == 0 && a.rank <= a.kd && a.rank <= 512,
              "latent attention on the tensor cores: keys of %d and values of %d must be multiples of 16, values at most 512 and "
              "inside the key", a.kd, a.rank);
  TIE_REQUIRE(latent_smem(a.kd) <= 200 * 1024, "latent attention on the tensor cores: keys of %d exceed shared memory", a.kd);
  TIE_REQUIRE(a.q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(a.q) % 16 == 0 && reinterpret_cast<uintptr_t>(a.keys) % 16 == 0,
              "latent attention on the tensor cores: queries and keys must be 16-byte aligned");
  TIE_REQUIRE(a.page_size > 0 && a.max_blocks > 0 && a.window >= 0, "latent attention: bad page geometry");
  return kOk;
}

}  // namespace tie

using namespace tie;

// Whether the tensor-core kernel takes these sizes (the part asks before it chooses a path).
TIE_API int tie_attention_latent_mma_takes(int kd, int rank) {
  return kd > 0 && kd % 16 == 0 && rank > 0 && rank % 16 == 0 && rank <= kd && rank <= 512 && latent_smem(kd) <= 200 * 1024;
}

// The first n_seqs sequences of the step bring several tokens each (their rows come first); max_queries is the most.
TIE_API int tie_attention_latent_prompt(const void* q, long long q_stride, const void* keys, void* out, const int* query_start,
                                        const int* context_lens, const int* block_tables, int max_blocks, int n_seqs,
                                        int max_queries, int heads, int kd, int rank, int page_size, int window, float scale,
                                        cudaStream_t s) {
  LatentArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(keys), static_cast<__nv_bfloat16*>(out),
               query_start, context_lens, block_tables, q_stride, max_blocks, heads, kd, rank, page_size, window,
               scale * 1.4426950408889634f, nullptr, 0, 0, 0, nullptr};
  if (const int st = check_latent(a)) return st;
  if (n_seqs <= 0 || max_queries <= 0) return kOk;
  const int hc = heads < kLatRows ? heads : kLatRows, bq = kLatRows / hc;
  TIE_REQUIRE(n_seqs <= 65535, "latent attention: %d sequences exceed the grid", n_seqs);
  return launch_latent<false>(a, dim3(ceil_div(max_queries, bq), n_seqs, ceil_div(heads, hc)), s);
}

// Sequences of seq_list bring one token each; scratch [n_list, heads, max_splits, rank + 2] is what tie_attention_merge reads.
TIE_API int tie_attention_latent_split(const void* q, long long q_stride, const void* keys, const int* query_start,
                                       const int* context_lens, const int* block_tables, int max_blocks, int heads, int kd,
                                       int rank, int page_size, int window, float scale, const int* seq_list, int n_list,
                                       int split_keys, int max_splits, float* scratch, cudaStream_t s) {
  LatentArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(keys), nullptr, query_start, context_lens,
               block_tables, q_stride, max_blocks, heads, kd, rank, page_size, window, scale * 1.4426950408889634f, seq_list,
               n_list, split_keys, max_splits, scratch};
  if (const int st = check_latent(a)) return st;
  TIE_REQUIRE(split_keys > 0 && max_splits > 0 && max_splits <= 256 && scratch != nullptr && n_list <= 65535,
              "latent attention split: bad split geometry");
  if (n_list <= 0) return kOk;
  const int hc = heads < kLatRows ? heads : kLatRows;
  return launch_latent<true>(a, dim3(max_splits, n_list, ceil_div(heads, hc)), s);
}

// bfloat16 tensor-core form of the attention without a softmax (mma.sync m16n8k16, float32
// accumulators): one CTA of four or eight warps works on up to 64 or 128 (token, head-of-group)
// rows of one sequence and one key/value head (16 rows a warp; the wider form for prompt
// portions, where it halves what a key tile costs per row); key tiles of 64 keys are anchored at absolute position 0,
// so the tiles a row adds up, and their order, depend on the row's position alone (a tile in
// which a row sees nothing adds exact zeros).  Scores are float32 sums of exact bfloat16
// products, the sigmoid is float32, the weights are rounded to bfloat16 for the product with
// the values, which accumulates in float32.  Keys and values of a tile arrive by cp.async,
// two tiles deep.
//
// KSPLIT (tiles of at most 16 rows: decoded tokens): the four warps share the 16 rows and
// each takes 16 of a tile's 64 keys; at the end the warps' sums are added in warp order.  A
// token's key tiles (in the order they are walked) are cut into chunks of `chunk_tiles`, a CTA
// per chunk (blockIdx.z), each writing its float32 sums; a second kernel adds a row's chunks
// in chunk order.  A row's sum over its keys is then associated differently than in the other
// form (by roundings of float32), again in a way that depends on its position alone.
#pragma once

#include <cuda_pipeline.h>

#include "source.cuh"

namespace sa_mma {

constexpr int KT = 64;        // keys of a tile
constexpr int PAD = 8;        // bfloat16 elements of padding per shared-memory row

__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 1 / (1 + 2^(-x log2 e)) on the special-function unit (relative error about 1e-6, far below
// the bfloat16 step of the weight it becomes)
__device__ __forceinline__ float sigmoid_fast(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}
// 16 bytes global -> shared; `valid` false: zeros
__device__ __forceinline__ void copy16(void* dst, const void* src, bool valid) {
  if (valid) __pipeline_memcpy_async(dst, src, 16);
  else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
}

// tiles: int32 [n][3] = (sequence of the step, first token of the tile in the step, tokens).
// NV16: value columns in units of 16 the accumulators are sized for (VD <= 16 * NV16).
// ROWS: query rows of a CTA (64 or 128; 16 with KSPLIT, on four warps).
template <int NV16, int ROWS, bool KSPLIT>
__global__ void __launch_bounds__(KSPLIT ? 128 : ROWS * 2)
sigmoid_attention_mma_kernel(const __nv_bfloat16* q, __nv_bfloat16* out, const __nv_bfloat16* cache,
                             const int* block_table, int bt_width, const int* positions, const int* seq_lens,
                             const int* tiles, const float* head_bias, int Hq, int Hkv, int D, int VD,
                             int page_size, float scale, int window, int keep_first, float* partial,
                             int chunk_tiles, int max_chunks) {
  extern __shared__ __align__(16) unsigned char sam_smem[];
  const int R = Hq / Hkv;
  const int qs = D + PAD, vs = VD + PAD;                 // row strides in elements
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sam_smem);            // [ROWS][qs]
  __nv_bfloat16* Ks = Qs + ROWS * qs;                                         // [2][KT][qs]
  __nv_bfloat16* Vs = Ks + 2 * KT * qs;                                       // [2][KT][vs]
  // where the rows of a key tile lie in the cache (elements; -1: past the sequence's keys),
  // found one tile ahead of the copies that use them
  __shared__ long long k_off[2][KT], v_off[2][KT];
  pdl_prologue();
  const int tile = blockIdx.x, g = blockIdx.y;
  const int b = tiles[3 * tile], t0 = tiles[3 * tile + 1], count = tiles[3 * tile + 2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int kv_len = seq_lens[b];
  const int pos0 = positions[t0];                        // the tile's tokens are consecutive positions
  const int pos_last = pos0 + count - 1;
  const int rows_used = count * R;
  const int* bt = block_table + (long long)b * bt_width;
  const long long page_elems = (long long)Hkv * page_size * (D + VD);

  // key tiles: those of the kept first keys below the window, then those of the windows
  const int lo_min = window > 0 ? (pos0 - window + 1 > 0 ? pos0 - window + 1 : 0) : 0;
  const int w_first = lo_min / KT, w_last = pos_last / KT;
  int kept_tiles = 0;
  if (window > 0 && keep_first > 0) {
    kept_tiles = (keep_first + KT - 1) / KT;
    if (kept_tiles > w_first) kept_tiles = w_first;
  }
  const int n_tiles = kept_tiles + (w_last - w_first + 1);
  // the tiles this CTA walks: all of them, or its chunk of them
  const int chunk = (KSPLIT && partial != nullptr) ? blockIdx.z : 0;
  const int it_begin = chunk * ((KSPLIT && partial != nullptr) ? chunk_tiles : 0);
  const int it_end = (KSPLIT && partial != nullptr && it_begin + chunk_tiles < n_tiles) ? it_begin + chunk_tiles
                                                                                      : n_tiles;
  if (it_begin >= n_tiles) return;          // (the whole CTA: no such chunk at this position)

  // Q rows: row r = token r / R, head g * R + r % R
  const int dchunks = D / 8;
  for (int idx = threadIdx.x; idx < ROWS * dchunks; idx += blockDim.x) {
    const int r = idx / dchunks, ch = idx - r * dchunks;
    const bool ok = r < rows_used;
    const int tl = ok ? r / R : 0, hh = ok ? r % R : 0;
    copy16(Qs + r * qs + ch * 8, q + ((long long)(t0 + tl) * Hq + g * R + hh) * D + ch * 8, ok);
  }
  auto tile_at = [&](int it) { return it < kept_tiles ? it : w_first + (it - kept_tiles); };

  const int vchunks = VD / 8;
  auto find_rows = [&](int it) {          // by the first KT threads, for tile `it` (if there is one)
    if (threadIdx.x < KT && it < it_end) {
      const int j = tile_at(it) * KT + threadIdx.x;
      long long ko = -1, vo = -1;
      if (j < kv_len) {
        const long long base = (long long)bt[j / page_size] * page_elems;
        const long long r = (long long)g * page_size + j % page_size;
        ko = base + r * D;
        vo = base + (long long)Hkv * page_size * D + r * VD;
      }
      k_off[it & 1][threadIdx.x] = ko;
      v_off[it & 1][threadIdx.x] = vo;
    }
  };
  auto load_tile = [&](int it, int stage) {
    __nv_bfloat16* kd = Ks + stage * KT * qs;
    __nv_bfloat16* vd = Vs + stage * KT * vs;
    for (int idx = threadIdx.x; idx < KT * dchunks; idx += blockDim.x) {
      const int jj = idx / dchunks, ch = idx - jj * dchunks;
      const long long off = k_off[stage][jj];
      copy16(kd + jj * qs + ch * 8, cache + (off < 0 ? 0 : off) + ch * 8, off >= 0);
    }
    for (int idx = threadIdx.x; idx < KT * vchunks; idx += blockDim.x) {
      const int jj = idx / vchunks, ch = idx - jj * vchunks;
      const long long off = v_off[stage][jj];
      copy16(vd + jj * vs + ch * 8, cache + (off < 0 ? 0 : off) + ch * 8, off >= 0);
    }
    __pipeline_commit();
  };

  // this thread's two rows: warp * 16 + gid and + 8
  int row_pos[2];
  float row_bias[2];
  const int row_base = KSPLIT ? 0 : warp * 16;         // the first of this warp's 16 rows
  const int key_base = KSPLIT ? warp * 16 : 0;         // the first of this warp's keys in a tile
  constexpr int NKT = KSPLIT ? 2 : KT / 8;             // 8-key blocks of a tile this warp works on
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_base + gid + 8 * h;
    const bool ok = r < rows_used;
    row_pos[h] = ok ? pos0 + r / R : -1;               // -1: sees nothing
    row_bias[h] = (ok && head_bias != nullptr) ? head_bias[g * R + r % R] : 0.f;
  }
  // positions of the warp's rows (for skipping tiles none of them sees)
  const int wr0 = row_base, wr1 = row_base + 15 < rows_used - 1 ? row_base + 15 : rows_used - 1;
  const bool warp_has_rows = wr0 < rows_used;
  const int wpos_first = pos0 + wr0 / R, wpos_last = warp_has_rows ? pos0 + wr1 / R : -1;

  float o[NV16 * 2][4];
#pragma unroll
  for (int n = 0; n < NV16 * 2; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  find_rows(it_begin);
  find_rows(it_begin + 1);
  __syncthreads();
  load_tile(it_begin, it_begin & 1);
  for (int it = it_begin; it < it_end; ++it) {
    const int stage = it & 1;
    if (it + 1 < it_end) {
      load_tile(it + 1, stage ^ 1);
      find_rows(it + 2);        // into this tile's entries: its copies were issued a round ago
      __pipeline_wait_prior(1);
    } else {
      __pipeline_wait_prior(0);
    }
    __syncthreads();
    const int k0 = tile_at(it) * KT;
    // does any row of this warp see a key of this tile?
    bool needed = warp_has_rows && k0 <= wpos_last;
    if (needed && window > 0) {
      const int tile_last = k0 + KT - 1;
      const bool in_window = tile_last > wpos_first - window;      // some key within the first row's window or later
      const bool in_kept = k0 < keep_first;
      needed = in_window || in_kept;
    }
    if (needed) {
      const __nv_bfloat16* kd = Ks + stage * KT * qs;
      const __nv_bfloat16* vd = Vs + stage * KT * vs;
      float s[NKT][4];
#pragma unroll
      for (int n = 0; n < NKT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a0, a1, a2, a3;
        ldsm_x4(a0, a1, a2, a3, Qs + (row_base + (lane & 15)) * qs + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int np = 0; np < NKT / 2; ++np) {
          unsigned b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3,
                  kd + (key_base + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * qs + kk * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * np], a0, a1, a2, a3, b0, b1);
          mma_bf16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      // weights: sigmoid(score * scale + bias) where the row sees the key, else 0
      unsigned p[NKT][2];
#pragma unroll
      for (int n = 0; n < NKT; ++n) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float w[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = k0 + key_base + n * 8 + tig * 2 + e;
            const int i = row_pos[h];
            const bool sees = j <= i && (window <= 0 || i - j < window || j < keep_first);
            w[e] = sees ? sigmoid_fast(__fmaf_rn(s[n][2 * h + e], scale, row_bias[h])) : 0.f;
          }
          p[n][h] = pack_bf16(w[0], w[1]);
        }
      }
#pragma unroll
      for (int kk = 0; kk < NKT / 2; ++kk) {
        const unsigned a0 = p[2 * kk][0], a1 = p[2 * kk][1], a2 = p[2 * kk + 1][0], a3 = p[2 * kk + 1][1];
#pragma unroll
        for (int np = 0; np < NV16; ++np) {
          if (np * 16 < VD) {
            unsigned b0, b1, b2, b3;
            ldsm_x4_trans(b0, b1, b2, b3,
                          vd + (key_base + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * vs + np * 16 + (lane >> 4) * 8);
            mma_bf16(o[2 * np], a0, a1, a2, a3, b0, b1);
            mma_bf16(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
    }
    __syncthreads();       // the stage is written again two tiles on
  }

  if constexpr (KSPLIT) {
    // the four warps' sums of the same 16 rows, added in warp order (the tiles' buffers are free:
    // the loop ended with a barrier)
    float* part = reinterpret_cast<float*>(Ks);          // [4 warps][16 rows][VD]
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int n = 0; n < NV16 * 2; ++n) {
        const int col = n * 8 + tig * 2;
        if (col < VD) {
          float* at = part + ((warp * 16) + gid + 8 * h) * VD + col;
          at[0] = o[n][2 * h];
          at[1] = o[n][2 * h + 1];
        }
      }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows_used * VD; idx += blockDim.x) {
      const int r = idx / VD, col = idx - r * VD;
      float v = part[r * VD + col];
#pragma unroll
      for (int w = 1; w < 4; ++w) v = __fadd_rn(v, part[(w * 16 + r) * VD + col]);
      const long long row = (long long)(t0 + r / R) * Hq + g * R + r % R;
      if (partial != nullptr) partial[(row * max_chunks + chunk) * VD + col] = v;
      else out[row * VD + col] = __float2bfloat16_rn(v);
    }
  } else {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + gid + 8 * h;
    if (r < rows_used) {
      __nv_bfloat16* dst = out + ((long long)(t0 + r / R) * Hq + g * R + r % R) * VD;
#pragma unroll
      for (int n = 0; n < NV16 * 2; ++n) {
        const int col = n * 8 + tig * 2;
        if (col < VD)
          *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[n][2 * h], o[n][2 * h + 1]);
      }
    }
  }
  }
}

// out[t, h, :] = the sum of the row's chunks in chunk order; a token at position p has
// ceil(tiles(p) / chunk_tiles) chunks, tiles(p) as the kernel above counts them.
__global__ void sigmoid_attention_merge_kernel(const float* partial, __nv_bfloat16* out, const int* positions,
                                               int Hq, int VD, int window, int keep_first, int chunk_tiles,
                                               int max_chunks) {
  pdl_prologue();
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  const int lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  const int w_first = lo / KT, w_last = pos / KT;
  int kept_tiles = 0;
  if (window > 0 && keep_first > 0) {
    kept_tiles = (keep_first + KT - 1) / KT;
    if (kept_tiles > w_first) kept_tiles = w_first;
  }
  const int n_tiles = kept_tiles + (w_last - w_first + 1);
  int chunks = (n_tiles + chunk_tiles - 1) / chunk_tiles;
  if (chunks > max_chunks) chunks = max_chunks;
  const long long row = (long long)t * Hq + h;
  for (int col = threadIdx.x; col < VD; col += blockDim.x) {
    float v = partial[(row * max_chunks) * VD + col];
    for (int c = 1; c < chunks; ++c) v = __fadd_rn(v, partial[(row * max_chunks + c) * VD + col]);
    out[row * VD + col] = __float2bfloat16_rn(v);
  }
}

static inline size_t smem_bytes(int D, int VD, int rows) {
  return sizeof(__nv_bfloat16) * ((size_t)rows * (D + PAD) + 2 * (size_t)KT * (D + PAD) + 2 * (size_t)KT * (VD + PAD));
}

template <int NV16, int ROWS, bool KSPLIT>
static int launch(const void* q, void* out, const void* cache, const int* block_table, int bt_width,
                  const int* positions, const int* seq_lens, const int* tiles, int num_tiles,
                  const float* head_bias, int Hq, int Hkv, int D, int VD, int page_size, float scale, int window,
                  int keep_first, float* partial, int chunk_tiles, int max_chunks, int num_tokens,
                  cudaStream_t st) {
  const size_t smem = smem_bytes(D, VD, ROWS);
  const bool chunked = KSPLIT && partial != nullptr;
  static DeviceOnce once;
  if (!once.done()) {
    if (cudaFuncSetAttribute(sigmoid_attention_mma_kernel<NV16, ROWS, KSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    once.mark();
  }
  dib_launch(sigmoid_attention_mma_kernel<NV16, ROWS, KSPLIT>, dim3(num_tiles, Hkv, chunked ? max_chunks : 1),
             dim3(KSPLIT ? 128 : ROWS * 2), smem, st, (const __nv_bfloat16*)q, (__nv_bfloat16*)out,
             (const __nv_bfloat16*)cache, block_table, bt_width, positions, seq_lens, tiles, head_bias, Hq, Hkv, D,
             VD, page_size, scale, window, keep_first, chunked ? partial : (float*)nullptr, chunk_tiles, max_chunks);
  DIB_CHECK_LAUNCH();
  if (chunked) {
    dib_launch(sigmoid_attention_merge_kernel, dim3(num_tokens, Hq), dim3(VD >= 128 ? 128 : 64), 0, st,
               (const float*)partial, (__nv_bfloat16*)out, positions, Hq, VD, window, keep_first, chunk_tiles,
               max_chunks);
    DIB_CHECK_LAUNCH();
  }
  return DIB_OK;
}

}  // namespace sa_mma

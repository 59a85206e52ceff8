// Attention without a softmax over a paged cache whose values may have another size than
// its keys: the weight of a visible key is sigmoid(q . k * scale + bias[head]), weights are
// not normalised over keys.  A query at position i sees key j <= i if i - j < window or
// j < keep_first (window 0: every j <= i).  Scores, weights and the weighted sum are float32;
// a (query, head) row adds its keys in ascending order of position, so its bits depend on
// its own position alone.
//
// Page layout: the keys of a page [Hkv, page_size, D], then its values [Hkv, page_size, Dv].
#include "sigmoid_attention_mma.cuh"
#include "source.cuh"

// Projection rows [q heads | k heads | v heads] plus a bias: q to q_out [T, Hq, D], k and v
// into the token's cache slot (slot = page * page_size + offset; negative: skip).
template <typename T>
__global__ void qkv_bias_cache_kernel(Source qkv, const float* bias, T* q_out, T* cache,
                                      const int* slot_mapping, int Hq, int Hkv, int D, int VD,
                                      int page_size, long long num_pages, int write_cache) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int nq = Hq * D, nk = Hkv * D, nv = Hkv * VD;
  const int width = nq + nk + nv;
  const long long page_elems = (long long)Hkv * page_size * (D + VD);
  const int slot = write_cache ? slot_mapping[t] : -1;
  const long long page = slot >= 0 ? slot / page_size : -1;
  const int off = slot >= 0 ? slot % page_size : 0;
  const bool ok = page >= 0 && page < num_pages;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = source_load(qkv, (long long)t * width + c);
    if (bias != nullptr) v = __fadd_rn(v, bias[c]);
    if (c < nq) {
      Elem<T>::store(q_out + (long long)t * nq + c, v);
    } else if (ok) {
      if (c < nq + nk) {
        const int g = (c - nq) / D, d = (c - nq) % D;
        Elem<T>::store(cache + page * page_elems + ((long long)g * page_size + off) * D + d, v);
      } else {
        const int g = (c - nq - nk) / VD, d = (c - nq - nk) % VD;
        Elem<T>::store(cache + page * page_elems + (long long)Hkv * page_size * D +
                           ((long long)g * page_size + off) * VD + d, v);
      }
    }
  }
}

constexpr int SA_TILE = 32;   // keys per tile of the kernel below

// One block per (token, kv head): the heads of the group share every key and value tile.
template <typename T>
__global__ void sigmoid_attention_kernel(const T* q, T* out, const T* cache, const int* block_table,
                                         int bt_width, const int* token_seq, const int* positions,
                                         const float* head_bias, int Hq, int Hkv, int D, int VD,
                                         int page_size, float scale, int window, int keep_first) {
  extern __shared__ float sa_smem[];
  const int R = Hq / Hkv;
  const int kstride = D + 1;
  float* qs = sa_smem;                 // [R][D]
  float* acc = qs + R * D;             // [R][VD]
  float* sc = acc + R * VD;            // [R][SA_TILE]
  float* kv = sc + R * SA_TILE;        // [SA_TILE][max(D + 1, VD)]
  pdl_prologue();
  const int t = blockIdx.x, g = blockIdx.y;
  const int i = positions[t], b = token_seq[t];
  const int* bt = block_table + (long long)b * bt_width;
  const long long page_elems = (long long)Hkv * page_size * (D + VD);
  for (int idx = threadIdx.x; idx < R * D; idx += blockDim.x)
    qs[idx] = Elem<T>::load(q + ((long long)t * Hq + (long long)g * R) * D + idx);
  for (int idx = threadIdx.x; idx < R * VD; idx += blockDim.x) acc[idx] = 0.f;
  const int lo = window > 0 ? (i - window + 1 > 0 ? i - window + 1 : 0) : 0;
  const int len_a = window > 0 ? (keep_first < lo ? keep_first : lo) : 0;   // kept first keys below the window
  const int n = len_a + (i - lo + 1);
  for (int n0 = 0; n0 < n; n0 += SA_TILE) {
    const int cnt = n - n0 < SA_TILE ? n - n0 : SA_TILE;
    __syncthreads();
    for (int idx = threadIdx.x; idx < cnt * D; idx += blockDim.x) {
      const int jj = idx / D, d = idx % D;
      const int m = n0 + jj;
      const int j = m < len_a ? m : lo + (m - len_a);
      const long long page = bt[j / page_size];
      kv[jj * kstride + d] =
          Elem<T>::load(cache + page * page_elems + ((long long)g * page_size + j % page_size) * D + d);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < R * SA_TILE; idx += blockDim.x) {
      const int r = idx / SA_TILE, jj = idx % SA_TILE;
      if (jj < cnt) {
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = __fmaf_rn(qs[r * D + d], kv[jj * kstride + d], dot);
        const float bias = head_bias != nullptr ? head_bias[g * R + r] : 0.f;
        sc[idx] = sigmoid_f32(__fmaf_rn(dot, scale, bias));
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < cnt * VD; idx += blockDim.x) {
      const int jj = idx / VD, d = idx % VD;
      const int m = n0 + jj;
      const int j = m < len_a ? m : lo + (m - len_a);
      const long long page = bt[j / page_size];
      kv[jj * VD + d] = Elem<T>::load(cache + page * page_elems + (long long)Hkv * page_size * D +
                                      ((long long)g * page_size + j % page_size) * VD + d);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < R * VD; idx += blockDim.x) {
      const int r = idx / VD, d = idx % VD;
      float a = acc[idx];
      for (int jj = 0; jj < cnt; ++jj) a = __fmaf_rn(sc[r * SA_TILE + jj], kv[jj * VD + d], a);
      acc[idx] = a;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < R * VD; idx += blockDim.x)
    Elem<T>::store(out + ((long long)t * Hq + (long long)g * R) * VD + idx, acc[idx]);
}

template <typename T>
static int launch_sigmoid_attention(const void* q, void* out, const void* cache, const int* block_table,
                                    int bt_width, const int* token_seq, const int* positions,
                                    const float* head_bias, int T_, int Hq, int Hkv, int D, int VD,
                                    int page_size, float scale, int window, int keep_first,
                                    cudaStream_t st) {
  const int R = Hq / Hkv;
  const int wide = D + 1 > VD ? D + 1 : VD;
  const size_t smem = sizeof(float) * ((size_t)R * D + (size_t)R * VD + (size_t)R * SA_TILE + (size_t)SA_TILE * wide);
  if (smem > 200 * 1024) return DIB_BAD_SIZE;
  static DeviceOnce once;
  if (smem > 48 * 1024 || !once.done()) {
    if (cudaFuncSetAttribute(sigmoid_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess)
      return DIB_LAUNCH_FAILED;
    once.mark();
  }
  dib_launch(sigmoid_attention_kernel<T>, dim3(T_, Hkv), dim3(128), smem, st, (const T*)q, (T*)out,
             (const T*)cache, block_table, bt_width, token_seq, positions, head_bias, Hq, Hkv, D, VD,
             page_size, scale, window, keep_first);
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

extern "C" {

int dib_qkv_bias_cache(const void* qkv, int kind, int splits, long long stride, const float* bias,
                       void* q_out, void* cache, const int* slot_mapping, int T_, int Hq, int Hkv, int D,
                       int VD, int page_size, long long num_pages, int dtype, cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  if (Hq < 1 || Hkv < 1 || D < 1 || VD < 1 || page_size < 1) return DIB_BAD_SIZE;
  const Source s = make_source(qkv, kind, splits, stride);
  const int wc = cache != nullptr ? 1 : 0;
  if (dtype == 0)
    dib_launch(qkv_bias_cache_kernel<float>, dim3(T_), dim3(256), 0, st, s, bias, (float*)q_out, (float*)cache,
               slot_mapping, Hq, Hkv, D, VD, page_size, num_pages, wc);
  else if (dtype == 1)
    dib_launch(qkv_bias_cache_kernel<__nv_bfloat16>, dim3(T_), dim3(256), 0, st, s, bias,
               (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, slot_mapping, Hq, Hkv, D, VD, page_size,
               num_pages, wc);
  else return DIB_BAD_DTYPE;
  DIB_CHECK_LAUNCH();
  return DIB_OK;
}

int dib_sigmoid_attention(const void* q, void* out, const void* cache, const int* block_table, int bt_width,
                          const int* token_seq, const int* positions, const float* head_bias, int T_, int Hq,
                          int Hkv, int D, int VD, int page_size, float scale, int window, int keep_first,
                          int dtype, cudaStream_t st) {
  if (T_ == 0) return DIB_OK;
  if (Hq < 1 || Hkv < 1 || Hq % Hkv || D < 1 || VD < 1 || page_size < 1 || window < 0 || keep_first < 0 ||
      Hkv > 65535)
    return DIB_BAD_SIZE;
  if (dtype == 0)
    return launch_sigmoid_attention<float>(q, out, cache, block_table, bt_width, token_seq, positions, head_bias,
                                           T_, Hq, Hkv, D, VD, page_size, scale, window, keep_first, st);
  if (dtype == 1)
    return launch_sigmoid_attention<__nv_bfloat16>(q, out, cache, block_table, bt_width, token_seq, positions,
                                                   head_bias, T_, Hq, Hkv, D, VD, page_size, scale, window,
                                                   keep_first, st);
  return DIB_BAD_DTYPE;
}

// The bfloat16 tensor-core form.  tiles: int32 [num_tiles][3] on the device = (sequence, first token
// of the tile in the step, tokens), at most rows / (Hq / Hkv) tokens of consecutive positions each;
// rows: 64 or 128 query rows to a CTA (the same bits either way), or 16: tiles of decoded tokens,
// whose keys the CTA's four warps share.  With rows 16 and partial != null (float32
// [num_tokens, Hq, max_chunks, VD]; the tiles are then the step's first num_tokens tokens, one
// each): a CTA per chunk of chunk_tiles key tiles and a second kernel that adds the chunks.
// Takes D a multiple of 16 up to 256, VD a multiple of 16 up to 256, Hq / Hkv <= 64, 16-byte aligned
// pointers; -2 otherwise (the caller runs the kernel above).
int dib_sigmoid_attention_mma(const void* q, void* out, const void* cache, const int* block_table, int bt_width,
                              const int* positions, const int* seq_lens, const int* tiles, int num_tiles,
                              const float* head_bias, int Hq, int Hkv, int D, int VD, int page_size, float scale,
                              int window, int keep_first, int rows, float* partial, int chunk_tiles,
                              int max_chunks, cudaStream_t st) {
  if (num_tiles == 0) return DIB_OK;
  if (rows != 16 && rows != 64 && rows != 128) return DIB_BAD_SIZE;
  if (rows == 16 && Hq / Hkv > 16) return DIB_BAD_SIZE;
  if (partial != nullptr && (rows != 16 || chunk_tiles < 1 || max_chunks < 1 || max_chunks > 65535))
    return DIB_BAD_SIZE;
  if (Hq < 1 || Hkv < 1 || Hq % Hkv || Hq / Hkv > 64 || D < 16 || D % 16 || D > 256 || VD < 16 || VD % 16 ||
      VD > 256 || page_size < 1 || window < 0 || keep_first < 0 || Hkv > 65535)
    return DIB_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) & 15) return DIB_BAD_ALIGN;
  if (sa_mma::smem_bytes(D, VD, rows) > 200 * 1024) return DIB_BAD_SIZE;
#define SA_LAUNCH(NV)                                                                                            \
  return rows == 16                                                                                              \
             ? sa_mma::launch<NV, 16, true>(q, out, cache, block_table, bt_width, positions, seq_lens, tiles,    \
                                            num_tiles, head_bias, Hq, Hkv, D, VD, page_size, scale, window,      \
                                            keep_first, partial, chunk_tiles, max_chunks, num_tiles, st)         \
         : rows == 64                                                                                            \
             ? sa_mma::launch<NV, 64, false>(q, out, cache, block_table, bt_width, positions, seq_lens, tiles,   \
                                             num_tiles, head_bias, Hq, Hkv, D, VD, page_size, scale, window,     \
                                             keep_first, nullptr, 0, 1, 0, st)                                   \
             : sa_mma::launch<NV, 128, false>(q, out, cache, block_table, bt_width, positions, seq_lens, tiles,  \
                                              num_tiles, head_bias, Hq, Hkv, D, VD, page_size, scale, window,    \
                                              keep_first, nullptr, 0, 1, 0, st)
  if (VD <= 64) SA_LAUNCH(4);
  if (VD <= 128) SA_LAUNCH(8);
  if (VD <= 192) SA_LAUNCH(12);
  SA_LAUNCH(16);
#undef SA_LAUNCH
}

}  // extern "C"

// Attention whose weights are sigmoids, not a softmax: the weight of a visible key is
//   sigmoid(q . k * scale + bias[head]),
// a number per query head added to the score, and the weights are not normalised over the keys, so the
// output is a plain sum: no running maximum, no denominator, and the parts of a split key range simply add.
//
// Values may be cached ROTATED by their own position (pairs of dims turned by position * freq, all value
// dims); each head's sum is then turned back by the query's position (by -position * freq) before it
// leaves: the weight of a value then depends on the distance between the two positions as well. The turn
// back is done here on the float32 sum.
//
// The general kernel: one warp per (token, query head, split of the key range), any head size that is a
// multiple of 8 up to 512, float32 or bfloat16 pages. Keys are walked 32 at a time in position order;
// a token's result depends only on its own query and the keys it reads.
#include "api.h"
#include "common.cuh"

namespace {

// Turn the row back: pair m of the first 2 * pairs dims by -pos * freq[m]; (u, v) -> (u c + v s, v c - u s).
// `row` holds the head's sum in shared memory; every lane writes its own dims.
template <typename T>
__device__ __forceinline__ void unrotate_store(const float* row, T* orow, int hd, int pos, const float* inv_freq,
                                               int pairs, int interleaved, int lane, int step) {
  for (int d = lane; d < hd; d += step) {
    float y = row[d];
    if (inv_freq && d < 2 * pairs) {
      const int m = interleaved ? (d >> 1) : (d < pairs ? d : d - pairs);
      float sn, cs;
      sincosf((float)pos * inv_freq[m], &sn, &cs);
      const bool first = interleaved ? !(d & 1) : d < pairs;
      const float other = row[interleaved ? (d ^ 1) : (first ? d + pairs : d - pairs)];
      y = first ? y * cs + other * sn : y * cs - other * sn;
    }
    orow[d] = hb::from_f32<T>(y);
  }
}

template <typename T, int kMaxDimsPerLane>
__global__ void sigmoid_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                         const T* __restrict__ v_pages, const int* __restrict__ block_table,
                                         int table_stride, const int* __restrict__ seq_of_token,
                                         const int* __restrict__ positions, const float* __restrict__ head_bias,
                                         const float* __restrict__ v_inv_freq, int v_pairs, int v_interleaved,
                                         T* __restrict__ out, int n_tokens, int nh, int nkv, int hd, int page_size,
                                         int chunk, int window, float scale, int split_size, int max_splits,
                                         float* __restrict__ part_acc) {
  extern __shared__ float q_smem[];  // [warps][hd]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (wid >= (long long)n_tokens * nh * max_splits) return;
  const int split = (int)(wid % max_splits);
  const long long th = wid / max_splits;
  const int t = (int)(th / nh);
  const int h = (int)(th - (long long)t * nh);
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  int lo = 0;
  if (chunk > 0) lo = (pos / chunk) * chunk;
  if (window > 0 && pos - window + 1 > lo) lo = pos - window + 1;
  int hi = pos;
  if (max_splits > 1) {
    lo += split * split_size;            // a function of the token's own visible range only
    hi = min(pos, lo + split_size - 1);
  }
  float* qs = q_smem + warp * hd;
  const T* qrow = q + ((size_t)t * nh + h) * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = hb::to_f32(qrow[d]) * scale;
  __syncwarp();
  const float bias = head_bias ? head_bias[h] : 0.f;

  float acc[kMaxDimsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] = 0.f;

  for (int base = lo; base <= hi; base += 32) {
    const int key = base + lane;
    float p = 0.f;
    int page = -1;
    if (key <= hi) {
      page = table[key / page_size];
      if (page >= 0) {
        const T* krow = k_pages + (((size_t)page * nkv + kvh) * page_size + (key % page_size)) * hd;
        float dot = 0.f;
        for (int d = 0; d < hd; d += 8) {
          float kv[8];
          hb::load8(krow + d, kv);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot += qs[d + e] * kv[e];
        }
        p = 1.f / (1.f + expf(-(dot + bias)));
      }
    }
    const int count = min(32, hi - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int pg = __shfl_sync(0xffffffffu, page, j);
      if (pg < 0) continue;
      const T* vrow = v_pages + (((size_t)pg * nkv + kvh) * page_size + ((base + j) % page_size)) * hd;
#pragma unroll
      for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] += pj * hb::to_f32(vrow[d]);
      }
    }
  }
  if (max_splits > 1) {
    float* pa = part_acc + ((size_t)th * max_splits + split) * hd;     // a split beyond the range leaves zeros
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) pa[d] = acc[i];
    }
    return;
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) qs[d] = acc[i];
  }
  __syncwarp();
  unrotate_store<T>(qs, out + ((size_t)t * nh + h) * hd, hd, pos, v_inv_freq, v_pairs, v_interleaved, lane, 32);
}

// The splits of each (token, head) added in split order, then turned back. A block per (token, head).
template <typename T>
__global__ void sigmoid_merge_kernel(const float* __restrict__ part_acc, const int* __restrict__ positions,
                                     const float* __restrict__ v_inv_freq, int v_pairs, int v_interleaved,
                                     T* __restrict__ out, int nh, int hd, int max_splits) {
  extern __shared__ float row[];    // [hd]
  const size_t th = blockIdx.x;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < max_splits; ++s) o += part_acc[(th * max_splits + s) * hd + d];
    row[d] = o;
  }
  __syncthreads();
  unrotate_store<T>(row, out + th * hd, hd, positions[th / nh], v_inv_freq, v_pairs, v_interleaved, threadIdx.x,
                    blockDim.x);
}

}  // namespace

extern "C" int hb_sigmoid_attention(const void* q, int dtype, const void* k_pages, const void* v_pages,
                                    const int* block_table, int table_stride, const int* seq_of_token,
                                    const int* positions, const float* head_bias, const float* v_inv_freq, int v_pairs,
                                    int v_interleaved, void* out, int n_tokens, int nh, int nkv, int hd, int page_size,
                                    int chunk, int window, float scale, int split_size, int max_splits,
                                    float* part_acc, cudaStream_t stream) {
  if (!q || !k_pages || !v_pages || !block_table || !seq_of_token || !positions || !out) return HB_ERR_BAD_ARG;
  if (max_splits < 1 || (max_splits > 1 && (split_size <= 0 || !part_acc))) return HB_ERR_BAD_ARG;
  if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || table_stride <= 0 || chunk < 0 ||
      window < 0 || v_pairs < 0 || 2 * v_pairs > hd)
    return HB_ERR_BAD_ARG;
  if (hd <= 0 || hd % 8 != 0 || hd > 512) return HB_ERR_UNSUPPORTED;
  if (!v_inv_freq) v_pairs = 0;
  if (n_tokens == 0) return HB_OK;
  const bool wide = hd > 256;
  const int warps_per_block = 4;
  const long long warps = (long long)n_tokens * nh * max_splits;
  const long long blocks = (warps + warps_per_block - 1) / warps_per_block;
  if (blocks > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;
  const size_t smem = (size_t)warps_per_block * hd * sizeof(float);
#define HB_SIGMOID_ATTENTION(T, DPL)                                                                            \
  sigmoid_attention_kernel<T, DPL><<<(int)blocks, warps_per_block * 32, smem, stream>>>(                        \
      (const T*)q, (const T*)k_pages, (const T*)v_pages, block_table, table_stride, seq_of_token, positions,    \
      head_bias, v_inv_freq, v_pairs, v_interleaved, (T*)out, n_tokens, nh, nkv, hd, page_size, chunk, window,  \
      scale, split_size, max_splits, part_acc)
  if (dtype == HB_DTYPE_F32) {
    if (wide) HB_SIGMOID_ATTENTION(float, 16); else HB_SIGMOID_ATTENTION(float, 8);
  } else if (dtype == HB_DTYPE_BF16) {
    if (wide) HB_SIGMOID_ATTENTION(__nv_bfloat16, 16); else HB_SIGMOID_ATTENTION(__nv_bfloat16, 8);
  } else {
    return HB_ERR_BAD_ARG;
  }
#undef HB_SIGMOID_ATTENTION
  HB_LAUNCH_CHECK();
  if (max_splits > 1) {
    const size_t msmem = (size_t)hd * sizeof(float);
    if (dtype == HB_DTYPE_F32)
      sigmoid_merge_kernel<float><<<n_tokens * nh, 128, msmem, stream>>>(part_acc, positions, v_inv_freq, v_pairs,
                                                                         v_interleaved, (float*)out, nh, hd, max_splits);
    else
      sigmoid_merge_kernel<__nv_bfloat16><<<n_tokens * nh, 128, msmem, stream>>>(
          part_acc, positions, v_inv_freq, v_pairs, v_interleaved, (__nv_bfloat16*)out, nh, hd, max_splits);
    HB_LAUNCH_CHECK();
  }
  return HB_OK;
}

extern "C" int hb_sigmoid_merge(const float* part_acc, const int* positions, const float* v_inv_freq, int v_pairs,
                                int v_interleaved, void* out, int dtype, int n_tokens, int nh, int hd, int max_splits,
                                cudaStream_t stream) {
  if (!part_acc || !positions || !out || n_tokens < 0 || nh <= 0 || hd <= 0 || max_splits < 1 || v_pairs < 0 ||
      2 * v_pairs > hd)
    return HB_ERR_BAD_ARG;
  if (!v_inv_freq) v_pairs = 0;
  if (n_tokens == 0) return HB_OK;
  if ((long long)n_tokens * nh > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;
  const size_t msmem = (size_t)hd * sizeof(float);
  if (dtype == HB_DTYPE_F32)
    sigmoid_merge_kernel<float><<<n_tokens * nh, 128, msmem, stream>>>(part_acc, positions, v_inv_freq, v_pairs,
                                                                       v_interleaved, (float*)out, nh, hd, max_splits);
  else if (dtype == HB_DTYPE_BF16)
    sigmoid_merge_kernel<__nv_bfloat16><<<n_tokens * nh, 128, msmem, stream>>>(
        part_acc, positions, v_inv_freq, v_pairs, v_interleaved, (__nv_bfloat16*)out, nh, hd, max_splits);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

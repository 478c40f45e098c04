// Latent attention's own small steps. The cache of such a mixer holds one latent row per token, from
// which every head's keys and values are linear maps; attention itself runs on the latents with the
// key map folded into the query and the value map applied to the result, through the paged attention
// kernels (one shared "kv head" whose keys and values are the same rows).
//
//   latent_append:  c = x / sqrt(mean(x^2) + eps) * w  (float32), written to the token's place in its page,
//                   zero-filled up to the page's row length
//                   With a rotated key part (rot_pairs > 0): the 2 * rot_pairs inputs behind the first `rank`
//                   are not normed; they are rotated by the token's position (pairs (i, i + rot_pairs), or
//                   (2i, 2i + 1); cos and sin times rot_mul) and written behind the latent, so a row is
//                   [c | rotated key part | zeros].
//   rope_copy:      dst[t, h, :2 * pairs] = src[t, h, :2 * pairs] rotated by the token's position: the rotated
//                   part of every query head, put where the attention kernel reads it
//   rmsnorm_rows:   y = x / sqrt(mean(x^2) + eps) * w over rows that are column slices (a query latent)
//   head_gate:      out[t, h, :] = in[t, h, :] * sigmoid(g[t, h])
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ in, long long in_stride, const T* __restrict__ w, float eps,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                     const int* __restrict__ block_table, int table_stride, T* __restrict__ pages,
                                     int page_size, int rank, int row_len, const float* __restrict__ inv_freq,
                                     int rot_pairs, int interleaved, float rot_mul) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const T* row = in + (size_t)t * in_stride;
  float ss = 0.f;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) {
    const float v = hb::to_f32(row[j]);
    ss += v * v;
  }
  const float inv = rsqrtf(hb::block_sum(ss, scratch) / (float)rank + eps);
  const int pos = positions[t];
  const int page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_size];
  if (page < 0) return;
  T* dst = pages + ((size_t)page * page_size + (pos % page_size)) * row_len;
  for (int j = threadIdx.x; j < row_len; j += blockDim.x) {
    float y = 0.f;
    if (j < rank) {
      y = hb::to_f32(row[j]) * inv * hb::to_f32(w[j]);
    } else if (j < rank + 2 * rot_pairs) {
      const int d = j - rank;
      const int m = interleaved ? (d >> 1) : (d < rot_pairs ? d : d - rot_pairs);
      const bool first = interleaved ? !(d & 1) : d < rot_pairs;
      const float mine = hb::to_f32(row[j]);
      const float other = hb::to_f32(row[rank + (interleaved ? (d ^ 1) : (first ? d + rot_pairs : d - rot_pairs))]);
      float sn, cs;
      sincosf((float)pos * inv_freq[m], &sn, &cs);
      sn *= rot_mul; cs *= rot_mul;
      y = first ? mine * cs - other * sn : mine * cs + other * sn;
    }
    dst[j] = hb::from_f32<T>(y);
  }
}

// grid (tokens), a thread per (head, dim of the rotated part).
template <typename T>
__global__ void rope_copy_kernel(const T* __restrict__ src, long long src_row, long long src_head,
                                 T* __restrict__ dst, long long dst_row, long long dst_head,
                                 const int* __restrict__ positions, const float* __restrict__ inv_freq, int heads,
                                 int pairs, int interleaved, float rot_mul) {
  const size_t t = blockIdx.x;
  const int pos = positions[t];
  const int dims = 2 * pairs;
  for (int e = threadIdx.x; e < heads * dims; e += blockDim.x) {
    const int h = e / dims, d = e - h * dims;
    const int m = interleaved ? (d >> 1) : (d < pairs ? d : d - pairs);
    const bool first = interleaved ? !(d & 1) : d < pairs;
    const T* s = src + t * src_row + (size_t)h * src_head;
    const float mine = hb::to_f32(s[d]);
    const float other = hb::to_f32(s[interleaved ? (d ^ 1) : (first ? d + pairs : d - pairs)]);
    float sn, cs;
    sincosf((float)pos * inv_freq[m], &sn, &cs);
    sn *= rot_mul; cs *= rot_mul;
    dst[t * dst_row + (size_t)h * dst_head + d] = hb::from_f32<T>(first ? mine * cs - other * sn : mine * cs + other * sn);
  }
}

// y = x / sqrt(mean(x^2) + eps) * w for rows that may be column slices of a wider matrix. A block per row.
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ in, long long in_stride, const T* __restrict__ w, float eps,
                                    T* __restrict__ out, int width) {
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  const T* row = in + t * in_stride;
  float ss = 0.f;
  for (int j = threadIdx.x; j < width; j += blockDim.x) {
    const float x = hb::to_f32(row[j]);
    ss += x * x;
  }
  const float inv = 1.f / sqrtf(hb::block_sum(ss, scratch) / (float)width + eps);
  for (int j = threadIdx.x; j < width; j += blockDim.x)
    out[t * width + j] = hb::from_f32<T>(hb::to_f32(row[j]) * inv * hb::to_f32(w[j]));
}

template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ in, const T* __restrict__ gate, long long gate_stride,
                                 T* __restrict__ out, int heads, int dim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
    const int h = i / dim;
    const float g = hb::to_f32(gate[(size_t)t * gate_stride + h]);
    const size_t at = (size_t)t * heads * dim + i;
    out[at] = hb::from_f32<T>(hb::to_f32(in[at]) / (1.f + expf(-g)));
  }
}

}  // namespace

extern "C" int hb_latent_append(const void* in, int dtype, long long in_stride, const void* w, float eps,
                                const int* positions, const int* seq_of_token, const int* block_table,
                                int table_stride, void* pages, int page_size, int rank, int row_len, int n_tokens,
                                const float* inv_freq, int rot_pairs, int interleaved, float rot_mul,
                                cudaStream_t stream) {
  if (!in || !w || !positions || !seq_of_token || !block_table || !pages) return HB_ERR_BAD_ARG;
  if (!inv_freq) rot_pairs = 0;
  if (rank <= 0 || rot_pairs < 0 || row_len < rank + 2 * rot_pairs || page_size <= 0 || table_stride <= 0 ||
      n_tokens < 0 || in_stride < rank + 2 * rot_pairs)
    return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int threads = rank >= 256 ? 256 : (rank >= 128 ? 128 : 64);
  if (dtype == HB_DTYPE_F32)
    latent_append_kernel<float><<<n_tokens, threads, 0, stream>>>(
        (const float*)in, in_stride, (const float*)w, eps, positions, seq_of_token, block_table, table_stride,
        (float*)pages, page_size, rank, row_len, inv_freq, rot_pairs, interleaved, rot_mul);
  else if (dtype == HB_DTYPE_BF16)
    latent_append_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)w, eps, positions, seq_of_token, block_table,
        table_stride, (__nv_bfloat16*)pages, page_size, rank, row_len, inv_freq, rot_pairs, interleaved, rot_mul);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_rope_copy(const void* src, long long src_row, long long src_head, void* dst, long long dst_row,
                            long long dst_head, int dtype, const int* positions, const float* inv_freq, int n_tokens,
                            int heads, int pairs, int interleaved, float rot_mul, cudaStream_t stream) {
  if (!src || !dst || !positions || !inv_freq || n_tokens < 0 || heads <= 0 || pairs <= 0) return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int work = heads * 2 * pairs;
  const int threads = work >= 256 ? 256 : (work + 31) / 32 * 32;
  if (dtype == HB_DTYPE_F32)
    rope_copy_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)src, src_row, src_head, (float*)dst, dst_row,
                                                              dst_head, positions, inv_freq, heads, pairs, interleaved, rot_mul);
  else if (dtype == HB_DTYPE_BF16)
    rope_copy_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)src, src_row, src_head, (__nv_bfloat16*)dst, dst_row, dst_head, positions, inv_freq,
        heads, pairs, interleaved, rot_mul);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_head_gate(const void* in, const void* gate, long long gate_stride, void* out, int dtype,
                            int n_tokens, int heads, int dim, cudaStream_t stream) {
  if (!in || !gate || !out || heads <= 0 || dim <= 0 || n_tokens < 0 || gate_stride < heads) return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int threads = heads * dim >= 256 ? 256 : 128;
  if (dtype == HB_DTYPE_F32)
    head_gate_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)in, (const float*)gate, gate_stride,
                                                              (float*)out, heads, dim);
  else if (dtype == HB_DTYPE_BF16)
    head_gate_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)in, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, heads, dim);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_rmsnorm_rows(const void* in, int dtype, long long in_stride, const void* w, float eps, void* out,
                               int n_rows, int width, cudaStream_t stream) {
  if (!in || !w || !out || n_rows < 0 || width <= 0 || in_stride < width) return HB_ERR_BAD_ARG;
  if (n_rows == 0) return HB_OK;
  const int threads = width >= 256 ? 256 : (width >= 128 ? 128 : 64);
  if (dtype == HB_DTYPE_F32)
    rmsnorm_rows_kernel<float><<<n_rows, threads, 0, stream>>>((const float*)in, in_stride, (const float*)w, eps,
                                                               (float*)out, width);
  else if (dtype == HB_DTYPE_BF16)
    rmsnorm_rows_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
        (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)out, width);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

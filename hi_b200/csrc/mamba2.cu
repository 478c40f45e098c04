// The Mamba-2 mixer around its recurrence. With heads of vdim value channels, G groups of N state channels and
// one projection row per token laid out as [z: heads*vdim | x: heads*vdim | B: G*N | C: G*N | dt: heads]:
//
//   mamba2_prep   per token: causal convolution over time (taps [C, K] float32, last column the token's own,
//                 plus a bias per channel) and silu of the x | B | C channels (rows before the portion's first
//                 token come from the request's state); dt = softplus(dt + dt_bias), no clamp;
//                 decay = exp(-exp(A_log[h]) * dt), written out per state channel of the head;
//                 x (float32, for the skip), v = dt * x, k = B, q = C.
//                 The recurrence itself is the delta rule's kernel without its correction term
//                 (S <- decay * S + k v^T, o = S^T q; S [N, vdim] per head, a head reads its group's B and C),
//                 and the state's convolution rows are moved by hb_delta_conv_update.
//   mamba2_out    y = (o + D[h] * x) * silu(z); RMS norm of y in `parts` equal runs of channels, each by its own
//                 root mean square; times a weight per channel; rounded to the engine's dtype.
//
// Everything between the projection and the normed output is float32.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const void* p, int dtype, size_t i) {
  return dtype == HB_DTYPE_F32 ? reinterpret_cast<const float*>(p)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float silu1(float v) { return v / (1.f + expf(-v)); }

struct MambaPrepArgs {
  const void* proj;      // [N, ld]
  int proj_dtype;
  long long ld;
  int chan_off, dt_off;  // first column of the x | B | C channels, of dt
  const float* taps;     // [C, K]
  const float* conv_bias;  // [C]
  const float* state;    // [slots, state_stride]; the convolution's last K-1 inputs [K-1, C] at conv_off
  long long state_stride, conv_off;
  const float* dt_bias;  // [heads]
  const float* a_log;    // [heads]
  const int* cu_seqlens;
  const int* seq_of_token;
  const int* slots;
  float* x;              // [N, heads * vdim]
  float* v;              // [N, heads * vdim]   dt * x
  float* k;              // [N, G * N]          B
  float* q;              // [N, G * N]          C
  float* decay;          // [N, heads * N]
  int heads, groups, n_state, vdim, K;
};

// grid (tokens, groups of units), a warp per unit: a unit is one head's x channels (with its dt and decay) or one
// group's B or C channels.
__global__ void mamba2_prep_kernel(const MambaPrepArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int s = a.seq_of_token[t];
  const int start = a.cu_seqlens[s];
  const int local = t - start;
  const int inner = a.heads * a.vdim, gn = a.groups * a.n_state, C = inner + 2 * gn, K = a.K;
  const float* conv = a.state + (size_t)a.slots[s] * a.state_stride + a.conv_off;   // [K-1, C]
  const int units = a.heads + 2 * a.groups;
  for (int u = blockIdx.y * warps + warp; u < units; u += gridDim.y * warps) {
    const bool is_x = u < a.heads;
    const int len = is_x ? a.vdim : a.n_state;
    const int c0 = is_x ? u * a.vdim : inner + (u - a.heads) * a.n_state;
    float dt = 0.f;
    if (is_x) {
      const float z = ldf(a.proj, a.proj_dtype, (size_t)t * a.ld + a.dt_off + u) + a.dt_bias[u];
      dt = z > 20.f ? z : log1pf(expf(z));
      const float g = expf(-expf(a.a_log[u]) * dt);
      for (int i = lane; i < a.n_state; i += 32) a.decay[((size_t)t * a.heads + u) * a.n_state + i] = g;
    }
    for (int i = lane; i < len; i += 32) {
      const int c = c0 + i;
      float acc = a.conv_bias ? a.conv_bias[c] : 0.f;
      for (int j = 0; j < K; ++j) {
        const int rel = local - (K - 1) + j;
        const float xin = rel >= 0 ? ldf(a.proj, a.proj_dtype, (size_t)(start + rel) * a.ld + a.chan_off + c)
                                   : conv[(size_t)(K - 1 + rel) * C + c];
        acc += a.taps[(size_t)c * K + j] * xin;
      }
      const float y = silu1(acc);
      if (is_x) {
        a.x[(size_t)t * inner + c] = y;
        a.v[(size_t)t * inner + c] = dt * y;
      } else if (c < inner + gn) {
        a.k[(size_t)t * gn + (c - inner)] = y;
      } else {
        a.q[(size_t)t * gn + (c - inner - gn)] = y;
      }
    }
  }
}

// The same for sizes and offsets that are multiples of four: a thread takes four neighbouring channels of a unit with
// one 8-byte (bfloat16) or 16-byte load per tap row, and writes 16 bytes at a time.
__device__ __forceinline__ float4 ld4(const void* p, int dtype, size_t i) {
  if (dtype == HB_DTYPE_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}

template <int KT>      // taps known at compile time (0: any number)
__global__ void mamba2_prep_vec_kernel(const MambaPrepArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int s = a.seq_of_token[t];
  const int start = a.cu_seqlens[s];
  const int local = t - start;
  const int inner = a.heads * a.vdim, gn = a.groups * a.n_state, C = inner + 2 * gn;
  const int K = KT ? KT : a.K;
  const float* conv = a.state + (size_t)a.slots[s] * a.state_stride + a.conv_off;   // [K-1, C]
  const int units = a.heads + 2 * a.groups;
  for (int u = blockIdx.y * warps + warp; u < units; u += gridDim.y * warps) {
    const bool is_x = u < a.heads;
    const int len = is_x ? a.vdim : a.n_state;
    const int c0 = is_x ? u * a.vdim : inner + (u - a.heads) * a.n_state;
    float dt = 0.f;
    if (is_x) {
      const float z = ldf(a.proj, a.proj_dtype, (size_t)t * a.ld + a.dt_off + u) + a.dt_bias[u];
      dt = z > 20.f ? z : log1pf(expf(z));
      const float g = expf(-expf(a.a_log[u]) * dt);
      const float4 g4 = make_float4(g, g, g, g);
      float4* dst = reinterpret_cast<float4*>(a.decay + ((size_t)t * a.heads + u) * a.n_state);
      for (int i = lane; i < a.n_state / 4; i += 32) dst[i] = g4;
    }
    for (int i = lane * 4; i < len; i += 128) {
      const int c = c0 + i;
      float4 acc = *reinterpret_cast<const float4*>(a.conv_bias + c);
      if (KT == 4) {
        // four taps: a channel's taps are one 16-byte load, and all four rows are asked for before the first is used
        float4 tp[4], xin[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) tp[e] = *reinterpret_cast<const float4*>(a.taps + (size_t)(c + e) * 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int rel = local - 3 + j;
          xin[j] = rel >= 0 ? ld4(a.proj, a.proj_dtype, (size_t)(start + rel) * a.ld + a.chan_off + c)
                            : *reinterpret_cast<const float4*>(conv + (size_t)(3 + rel) * C + c);
        }
        acc.x += tp[0].x * xin[0].x + tp[0].y * xin[1].x + tp[0].z * xin[2].x + tp[0].w * xin[3].x;
        acc.y += tp[1].x * xin[0].y + tp[1].y * xin[1].y + tp[1].z * xin[2].y + tp[1].w * xin[3].y;
        acc.z += tp[2].x * xin[0].z + tp[2].y * xin[1].z + tp[2].z * xin[2].z + tp[2].w * xin[3].z;
        acc.w += tp[3].x * xin[0].w + tp[3].y * xin[1].w + tp[3].z * xin[2].w + tp[3].w * xin[3].w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j < K) {
            const int rel = local - (K - 1) + j;
            const float4 xin = rel >= 0 ? ld4(a.proj, a.proj_dtype, (size_t)(start + rel) * a.ld + a.chan_off + c)
                                        : *reinterpret_cast<const float4*>(conv + (size_t)(K - 1 + rel) * C + c);
            acc.x += a.taps[(size_t)c * K + j] * xin.x;
            acc.y += a.taps[(size_t)(c + 1) * K + j] * xin.y;
            acc.z += a.taps[(size_t)(c + 2) * K + j] * xin.z;
            acc.w += a.taps[(size_t)(c + 3) * K + j] * xin.w;
          }
        }
      }
      const float4 y = make_float4(silu1(acc.x), silu1(acc.y), silu1(acc.z), silu1(acc.w));
      if (is_x) {
        *reinterpret_cast<float4*>(a.x + (size_t)t * inner + c) = y;
        *reinterpret_cast<float4*>(a.v + (size_t)t * inner + c) = make_float4(dt * y.x, dt * y.y, dt * y.z, dt * y.w);
      } else if (c < inner + gn) {
        *reinterpret_cast<float4*>(a.k + (size_t)t * gn + (c - inner)) = y;
      } else {
        *reinterpret_cast<float4*>(a.q + (size_t)t * gn + (c - inner - gn)) = y;
      }
    }
  }
}

// grid (tokens, parts); a block norms one run of inner / parts channels.
template <typename T>
__global__ void mamba2_out_kernel(const float* __restrict__ o, const float* __restrict__ x, const void* __restrict__ z,
                                  int z_dtype, long long z_stride, const float* __restrict__ d_skip,
                                  const T* __restrict__ w, float eps, T* __restrict__ out, int inner, int vdim, int run) {
  __shared__ float scratch[33];
  const size_t t = blockIdx.x;
  const int c0 = blockIdx.y * run;
  float ss = 0.f;
  for (int i = threadIdx.x; i < run; i += blockDim.x) {
    const int c = c0 + i;
    const float y = (o[t * inner + c] + d_skip[c / vdim] * x[t * inner + c]) * silu1(ldf(z, z_dtype, t * z_stride + c));
    ss += y * y;
  }
  const float inv = rsqrtf(hb::block_sum(ss, scratch) / (float)run + eps);
  for (int i = threadIdx.x; i < run; i += blockDim.x) {
    const int c = c0 + i;
    const float y = (o[t * inner + c] + d_skip[c / vdim] * x[t * inner + c]) * silu1(ldf(z, z_dtype, t * z_stride + c));
    out[t * inner + c] = hb::from_f32<T>(y * inv * hb::to_f32(w[c]));
  }
}

// The same with four channels a thread and the gated row kept in shared memory between the two passes, so that o, x
// and z are read once: for runs that are a multiple of four and fit there.
template <typename T>
__global__ void mamba2_out_vec_kernel(const float* __restrict__ o, const float* __restrict__ x, const void* __restrict__ z,
                                      int z_dtype, long long z_stride, const float* __restrict__ d_skip,
                                      const T* __restrict__ w, float eps, T* __restrict__ out, int inner, int vdim, int run) {
  __shared__ float scratch[33];
  extern __shared__ float4 y_s[];      // [run / 4]
  const size_t t = blockIdx.x;
  const int c0 = blockIdx.y * run;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < run; i += blockDim.x * 4) {
    const int c = c0 + i;
    const float4 ov = *reinterpret_cast<const float4*>(o + t * inner + c);
    const float4 xv = *reinterpret_cast<const float4*>(x + t * inner + c);
    const float4 zv = ld4(z, z_dtype, t * z_stride + c);
    const float d = d_skip[c / vdim];                      // four neighbours lie in one head (vdim % 4 == 0)
    const float4 y = make_float4((ov.x + d * xv.x) * silu1(zv.x), (ov.y + d * xv.y) * silu1(zv.y),
                                 (ov.z + d * xv.z) * silu1(zv.z), (ov.w + d * xv.w) * silu1(zv.w));
    y_s[i >> 2] = y;
    ss += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
  }
  const float inv = rsqrtf(hb::block_sum(ss, scratch) / (float)run + eps);
  for (int i = threadIdx.x * 4; i < run; i += blockDim.x * 4) {
    const int c = c0 + i;
    const float4 y = y_s[i >> 2];
    T* dst = out + t * inner + c;
    dst[0] = hb::from_f32<T>(y.x * inv * hb::to_f32(w[c]));
    dst[1] = hb::from_f32<T>(y.y * inv * hb::to_f32(w[c + 1]));
    dst[2] = hb::from_f32<T>(y.z * inv * hb::to_f32(w[c + 2]));
    dst[3] = hb::from_f32<T>(y.w * inv * hb::to_f32(w[c + 3]));
  }
}

}  // namespace

extern "C" int hb_mamba2_prep(const void* proj, int proj_dtype, long long ld, int chan_off, int dt_off, const float* taps,
                              const float* conv_bias, const float* state, long long state_stride, long long conv_off,
                              const float* dt_bias, const float* a_log, const int* cu_seqlens, const int* seq_of_token,
                              const int* slots, float* x, float* v, float* k, float* q, float* decay, int n_tokens,
                              int heads, int groups, int n_state, int vdim, int taps_n, cudaStream_t stream) {
  if (!proj || !taps || !state || !dt_bias || !a_log || !cu_seqlens || !seq_of_token || !slots || !x || !v || !k || !q ||
      !decay)
    return HB_ERR_BAD_ARG;
  if (n_tokens < 0 || heads <= 0 || groups <= 0 || heads % groups || n_state <= 0 || vdim <= 0 || taps_n < 1)
    return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  MambaPrepArgs a;
  a.proj = proj; a.proj_dtype = proj_dtype; a.ld = ld; a.chan_off = chan_off; a.dt_off = dt_off; a.taps = taps;
  a.conv_bias = conv_bias; a.state = state; a.state_stride = state_stride; a.conv_off = conv_off; a.dt_bias = dt_bias;
  a.a_log = a_log; a.cu_seqlens = cu_seqlens; a.seq_of_token = seq_of_token; a.slots = slots; a.x = x; a.v = v; a.k = k;
  a.q = q; a.decay = decay; a.heads = heads; a.groups = groups; a.n_state = n_state; a.vdim = vdim; a.K = taps_n;
  const int units = heads + 2 * groups;
  const int warps = units < 4 ? units : 4;
  // a block finds its request's rows once and then takes units in turn: with many tokens few blocks a token, so
  // that the look-ups are shared by more work; with few tokens a block per group of units, to fill the GPU
  int gy = (units + warps - 1) / warps;
  const int want = (148 * 8 + n_tokens - 1) / n_tokens;
  if (gy > want) gy = want;
  if (gy > 64) gy = 64;
  const bool vec = conv_bias && vdim % 4 == 0 && n_state % 4 == 0 && ld % 4 == 0 && chan_off % 4 == 0 && conv_off % 4 == 0 &&
                   state_stride % 4 == 0 && taps_n <= 8;
  if (vec && taps_n == 4) mamba2_prep_vec_kernel<4><<<dim3(n_tokens, gy), warps * 32, 0, stream>>>(a);
  else if (vec) mamba2_prep_vec_kernel<0><<<dim3(n_tokens, gy), warps * 32, 0, stream>>>(a);
  else mamba2_prep_kernel<<<dim3(n_tokens, gy), warps * 32, 0, stream>>>(a);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_mamba2_out(const float* o, const float* x, const void* z, int z_dtype, long long z_stride,
                             const float* d_skip, const void* w, float eps, void* out, int dtype, int n_tokens, int heads,
                             int vdim, int parts, cudaStream_t stream) {
  if (!o || !x || !z || !d_skip || !w || !out || n_tokens < 0 || heads <= 0 || vdim <= 0 || parts <= 0)
    return HB_ERR_BAD_ARG;
  const int inner = heads * vdim;
  if (inner % parts || z_stride < inner || parts > 65535) return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int run = inner / parts;
  const int threads = run >= 1024 ? 256 : (run >= 128 ? 128 : (run + 31) / 32 * 32);
  const dim3 grid(n_tokens, parts);
  if (vdim % 4 == 0 && run % 4 == 0 && z_stride % 4 == 0 && (size_t)run * 4 <= 48 * 1024 &&
      (dtype == HB_DTYPE_F32 || dtype == HB_DTYPE_BF16)) {
    const int vthreads = run >= 1024 ? 256 : (run >= 512 ? 128 : (run / 4 + 31) / 32 * 32);
    const size_t smem = (size_t)run * sizeof(float);
    if (dtype == HB_DTYPE_F32)
      mamba2_out_vec_kernel<float><<<grid, vthreads, smem, stream>>>(o, x, z, z_dtype, z_stride, d_skip, (const float*)w, eps,
                                                                     (float*)out, inner, vdim, run);
    else
      mamba2_out_vec_kernel<__nv_bfloat16><<<grid, vthreads, smem, stream>>>(
          o, x, z, z_dtype, z_stride, d_skip, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)out, inner, vdim, run);
    HB_LAUNCH_CHECK();
    return HB_OK;
  }
  if (dtype == HB_DTYPE_F32)
    mamba2_out_kernel<float><<<grid, threads, 0, stream>>>(o, x, z, z_dtype, z_stride, d_skip, (const float*)w, eps,
                                                           (float*)out, inner, vdim, run);
  else if (dtype == HB_DTYPE_BF16)
    mamba2_out_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(o, x, z, z_dtype, z_stride, d_skip,
                                                                   (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)out,
                                                                   inner, vdim, run);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

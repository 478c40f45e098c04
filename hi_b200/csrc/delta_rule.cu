// The gated delta rule with one decay per head and key channel: a recurrent mixer whose per-request
// state is a matrix S [dim, vdim] per head in float32, plus the last (taps - 1) inputs of the short
// causal convolutions that q, k and v pass.
//
//   delta_prep         per token: convolution over time + silu of the q | k | v channels (the rows before the
//                      portion's first token come from the request's state), q and k to unit length per head
//                      (q also times dim^-1/2), beta = sigmoid(.), decay = exp(-exp(A_log) * softplus(a + dt_bias))
//   delta_conv_update  per request: the last (taps - 1) inputs of the portion replace the state's
//   delta_recurrence   per (request, head, group of value columns), token after token:
//                        S <- decay * S (rows);  u = beta * (v - S^T k);  S <- S + k u^T;  o = S^T q
//                      A thread owns one column of S, so nothing is exchanged between threads but k, q and the
//                      decay of the token, which the block stages in shared memory one token ahead.
//   delta_out_norm     o / sqrt(mean_vdim(o^2) + eps) * w * sigmoid(gate)   (or * silu(gate))
//   gla_prep           the inputs of the same recurrence without the correction (S <- decay * S + k v^T):
//                      q * dim^-1/2, k, v as float32 and decay = sigmoid(z + b)^(1 / tau) per key channel
//
// Everything here is float32 arithmetic; only the projections that come in and the normed output that
// goes out have the engine's dtype. The state of a request depends on its own tokens only and the order of
// the sums is fixed, so the result does not depend on how the tokens were cut into steps or batched.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float ldf(const void* p, int dtype, size_t i) {
  return dtype == HB_DTYPE_F32 ? reinterpret_cast<const float*>(p)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float sigmoid1(float v) { return 1.f / (1.f + expf(-v)); }

struct PrepArgs {
  const void* proj;          // [N, ld]: ... q | k | v channels from column `chan_off`, beta from `beta_off`
  int proj_dtype;
  long long ld;
  int chan_off, beta_off;
  const float* taps;         // [C, K]
  float* state;              // [slots, state_stride]
  long long state_stride, conv_off;
  const void* a_pre;         // [N, heads * dim]; with head_decay [N, heads]: one decay per head
  int a_dtype;
  int head_decay;
  const float* dt_bias;      // [heads * dim] ([heads] with head_decay)
  const float* a_log;        // [heads]
  const int* cu_seqlens;
  const int* seq_of_token;
  const int* slots;
  float* q;                  // [N, kvh * dim]
  float* k;                  // [N, kvh * dim]
  float* v;                  // [N, heads * vdim]
  float* beta;               // [N, heads]
  float* decay;              // [N, heads * dim]
  int heads, kvh, dim, vdim, K;
};

// grid (tokens, groups of units), a warp per unit: a unit is one q head, one k head (dim channels each) or
// one v head (vdim channels, with that head's beta and decays), so that a step of few tokens still fills
// the GPU. A lane reads back only what it wrote itself, so the warp needs no barrier.
__global__ void delta_prep_kernel(const PrepArgs a, int longest) {
  extern __shared__ float y_all[];     // [warps][longest]: a unit's channels after convolution and silu
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  float* y = y_all + (size_t)warp * longest;
  const int t = blockIdx.x;
  const int s = a.seq_of_token[t];
  const int start = a.cu_seqlens[s];
  const int local = t - start;
  const int qk = a.kvh * a.dim, C = 2 * qk + a.heads * a.vdim, K = a.K;
  const float* conv = a.state + (size_t)a.slots[s] * a.state_stride + a.conv_off;   // [K-1, C]
  const float qscale = 1.f / sqrtf((float)a.dim);
  const int units = 2 * a.kvh + a.heads;
  for (int u = blockIdx.y * warps + warp; u < units; u += gridDim.y * warps) {
    const bool is_v = u >= 2 * a.kvh;
    const int len = is_v ? a.vdim : a.dim;
    const int c0 = is_v ? 2 * qk + (u - 2 * a.kvh) * a.vdim : u * a.dim;
    float ss = 0.f;
    for (int i = lane; i < len; i += 32) {
      const int c = c0 + i;
      float acc = 0.f;
      for (int j = 0; j < K; ++j) {
        const int rel = local - (K - 1) + j;
        const float x = rel >= 0 ? ldf(a.proj, a.proj_dtype, (size_t)(start + rel) * a.ld + a.chan_off + c)
                                 : conv[(size_t)(K - 1 + rel) * C + c];
        acc += a.taps[(size_t)c * K + j] * x;
      }
      const float v = acc * sigmoid1(acc);
      y[i] = v;
      ss += v * v;
    }
    if (is_v) {
      const int h = u - 2 * a.kvh;
      for (int i = lane; i < len; i += 32) a.v[(size_t)t * a.heads * a.vdim + (size_t)h * a.vdim + i] = y[i];
      if (lane == 0)
        a.beta[(size_t)t * a.heads + h] = sigmoid1(ldf(a.proj, a.proj_dtype, (size_t)t * a.ld + a.beta_off + h));
      const float rate = expf(a.a_log[h]);
      if (a.head_decay) {
        // one decay for all key channels of the head, written out per channel: the recurrence reads rows of decays
        const float x = ldf(a.a_pre, a.a_dtype, (size_t)t * a.heads + h) + a.dt_bias[h];
        const float sp = x > 20.f ? x : log1pf(expf(x));
        const float g = expf(-rate * sp);
        for (int i = lane; i < a.dim; i += 32) a.decay[(size_t)t * a.heads * a.dim + (size_t)h * a.dim + i] = g;
      } else
      for (int i = lane; i < a.dim; i += 32) {
        const size_t at = (size_t)t * a.heads * a.dim + (size_t)h * a.dim + i;
        const float x = ldf(a.a_pre, a.a_dtype, at) + a.dt_bias[(size_t)h * a.dim + i];
        const float sp = x > 20.f ? x : log1pf(expf(x));
        a.decay[at] = expf(-rate * sp);
      }
    } else {
      const float inv = 1.f / sqrtf(hb::warp_sum(ss) + 1e-6f);
      const bool is_q = u < a.kvh;
      float* dst = is_q ? a.q + (size_t)t * qk + (size_t)u * a.dim : a.k + (size_t)t * qk + (size_t)(u - a.kvh) * a.dim;
      for (int i = lane; i < len; i += 32) dst[i] = is_q ? y[i] * inv * qscale : y[i] * inv;
    }
  }
}

__global__ void delta_conv_update_kernel(const void* proj, int proj_dtype, long long ld, int chan_off, float* state,
                                         long long state_stride, long long conv_off, const int* cu_seqlens,
                                         const int* slots, int C, int K) {
  const int s = blockIdx.x;
  const int start = cu_seqlens[s], n = cu_seqlens[s + 1] - start;
  if (n <= 0) return;
  float* conv = state + (size_t)slots[s] * state_stride + conv_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    // row i of the new state is input (n - (K-1) + i) of the portion; a negative one is row (n + i) of the
    // old state, which lies behind every row written so far
    for (int i = 0; i < K - 1; ++i) {
      const int rel = n - (K - 1) + i;
      conv[(size_t)i * C + c] = rel >= 0 ? ldf(proj, proj_dtype, (size_t)(start + rel) * ld + chan_off + c)
                                         : conv[(size_t)(n + i) * C + c];
    }
  }
}

struct RecurArgs {
  const float* q;       // [N, kvh * dim]
  const float* k;
  const float* v;       // [N, heads * vdim]
  const float* beta;    // [N, heads]
  const float* decay;   // [N, heads * dim]
  float* state;         // [slots, state_stride], S of head h at h * dim * vdim, row-major [dim, vdim]
  long long state_stride;
  const int* cu_seqlens;
  const int* slots;
  float* out;           // [N, heads * vdim]
  int heads, kvh, dim, vdim;
  int plain;            // 1: no correction, S <- decay * S + k v^T (beta is not read)
};

// Stage token t's k, q and decay rows (dim floats each) into buf[0..3*DIMP): k, q, g.
__device__ __forceinline__ void stage_token(const RecurArgs& a, int t, int head, int kvhead, float* buf, int dimp) {
  for (int i = threadIdx.x; i < dimp; i += blockDim.x) {
    const bool in = i < a.dim;
    buf[i] = in ? a.k[(size_t)t * a.kvh * a.dim + (size_t)kvhead * a.dim + i] : 0.f;
    buf[dimp + i] = in ? a.q[(size_t)t * a.kvh * a.dim + (size_t)kvhead * a.dim + i] : 0.f;
    buf[2 * dimp + i] = in ? a.decay[(size_t)t * a.heads * a.dim + (size_t)head * a.dim + i] : 1.f;
  }
}

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src) {      // both 16-byte aligned
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

constexpr int kRecurTokens = 8;     // tokens staged per chunk
constexpr int kRecurThreads = 64;   // two warps a block

// A column of S in the registers of SPLIT lanes of one warp, ROWS rows each: lane = part * (32 / SPLIT) + c
// holds rows part * ROWS + r (r < ROWS) of the warp's column c; rows beyond dim stay zero. dim <= ROWS * SPLIT.
// The dot products of a token are summed within a thread in two interleaved chains, then across
// the SPLIT lanes by a butterfly: the order is fixed by the kernel's form alone.
// The tokens' k, q, decay, v and beta come into shared memory in chunks of kRecurTokens by cp.async, the next
// chunk while this one is worked on, so the chain from token to token never waits for memory.
// Layout of a token in a chunk: k[DIMP] q[DIMP] g[DIMP] v[block's columns] beta, padded to 16 bytes.
template <int ROWS, int SPLIT>
__global__ void __launch_bounds__(kRecurThreads) delta_recurrence_reg_kernel(const RecurArgs a) {
  // a lane's rows lie side by side in shared memory, 4 floats of padding after each lane's run, so that a lane
  // reads them four at a time and the SPLIT runs of a warp fall into different banks
  constexpr int RP = ROWS + 4, DIMP = RP * SPLIT, WCOLS = 32 / SPLIT, BCOLS = WCOLS * (kRecurThreads / 32);
  constexpr int TB = kRecurTokens, TOK = 3 * DIMP + (BCOLS + 4) / 4 * 4;
  extern __shared__ __align__(16) float sm[];     // [2][TB][TOK]
  const int head = blockIdx.y, seq = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane / WCOLS;
  const int bcol = warp * WCOLS + (lane % WCOLS);
  const int col0 = blockIdx.x * BCOLS;
  const int col = col0 + bcol;
  const bool active = col < a.vdim;
  const int kvhead = head / (a.heads / a.kvh);
  const int first = a.cu_seqlens[seq], last = a.cu_seqlens[seq + 1];
  if (first >= last) return;
  const int dim = a.dim;
  float* S = a.state + (size_t)a.slots[seq] * a.state_stride + (size_t)head * dim * a.vdim;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = part * ROWS + r;
    s[r] = (active && i < dim) ? S[(size_t)i * a.vdim + col] : 0.f;
  }
  // what no copy ever writes: rows beyond dim (k = q = 0, decay 1) and columns beyond vdim (v = 0)
  for (int e = threadIdx.x; e < 2 * TB * TOK; e += kRecurThreads) {
    const int f = e % TOK;
    sm[e] = (f >= 2 * DIMP && f < 3 * DIMP) ? 1.f : 0.f;
  }
  __syncthreads();
  const int bcols = min(BCOLS, a.vdim - col0);
  const bool wide = (dim & 3) == 0;                             // rows of k, q, decay in 16-byte pieces
  const bool wide_v = (a.vdim & 3) == 0 && (bcols & 3) == 0;
  auto stage = [&](int t0, int buf) {
    const int cnt = min(TB, last - t0);
    float* dst = sm + (size_t)buf * TB * TOK;
    const size_t qk_row = (size_t)a.kvh * dim, g_row = (size_t)a.heads * dim, v_row = (size_t)a.heads * a.vdim;
    if (wide) {
      const int per = dim >> 2;
      for (int e = threadIdx.x; e < cnt * per; e += kRecurThreads) {
        const int tok = e / per, i = (e - tok * per) << 2;
        float* d = dst + tok * TOK + (i / ROWS) * RP + (i % ROWS);
        cp_async16(d, a.k + (size_t)(t0 + tok) * qk_row + (size_t)kvhead * dim + i);
        cp_async16(d + DIMP, a.q + (size_t)(t0 + tok) * qk_row + (size_t)kvhead * dim + i);
        cp_async16(d + 2 * DIMP, a.decay + (size_t)(t0 + tok) * g_row + (size_t)head * dim + i);
      }
    } else {
      for (int e = threadIdx.x; e < cnt * dim; e += kRecurThreads) {
        const int tok = e / dim, i = e - tok * dim;
        float* d = dst + tok * TOK + (i / ROWS) * RP + (i % ROWS);
        cp_async4(d, a.k + (size_t)(t0 + tok) * qk_row + (size_t)kvhead * dim + i);
        cp_async4(d + DIMP, a.q + (size_t)(t0 + tok) * qk_row + (size_t)kvhead * dim + i);
        cp_async4(d + 2 * DIMP, a.decay + (size_t)(t0 + tok) * g_row + (size_t)head * dim + i);
      }
    }
    if (wide_v) {
      const int per = bcols >> 2;
      for (int e = threadIdx.x; e < cnt * per; e += kRecurThreads) {
        const int tok = e / per, c = (e - tok * per) << 2;
        cp_async16(dst + tok * TOK + 3 * DIMP + c, a.v + (size_t)(t0 + tok) * v_row + (size_t)head * a.vdim + col0 + c);
      }
    } else {
      for (int e = threadIdx.x; e < cnt * bcols; e += kRecurThreads) {
        const int tok = e / bcols, c = e - tok * bcols;
        cp_async4(dst + tok * TOK + 3 * DIMP + c, a.v + (size_t)(t0 + tok) * v_row + (size_t)head * a.vdim + col0 + c);
      }
    }
    if (!a.plain)
      for (int tok = threadIdx.x; tok < cnt; tok += kRecurThreads)
        cp_async4(dst + tok * TOK + 3 * DIMP + BCOLS, a.beta + (size_t)(t0 + tok) * a.heads + head);
  };
  stage(first, 0);
  cp_async_commit();
  int buf = 0;
  for (int t0 = first; t0 < last; t0 += TB, buf ^= 1) {
    const bool more = t0 + TB < last;
    if (more) stage(t0 + TB, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();          // everything but the group just committed: this chunk is in
    __syncthreads();
    const int cnt = min(TB, last - t0);
#pragma unroll 2      // the next token's loads do not wait for this token's update
    for (int tok = 0; tok < cnt; ++tok) {
      const float* base = sm + ((size_t)buf * TB + tok) * TOK;
      const float* cur = base + part * RP;
      const float vj = base[3 * DIMP + bcol];
      const float bt = base[3 * DIMP + BCOLS];
      // One pass gives all three dot products of the token over the decayed column s' = g * s:
      //   s'.k (for u), s'.q and k.q, since the read-out of the updated column is (s' + k u).q = s'.q + u (k.q).
      // One butterfly carries the three sums; the update s = s' + k u follows with nothing waiting on it
      // but the next token.
      float kk[ROWS];
      float ak[2] = {0.f, 0.f}, aq[2] = {0.f, 0.f}, akq[2] = {0.f, 0.f};
#pragma unroll
      for (int r4 = 0; r4 < ROWS; r4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(cur + r4);
        const float4 q4 = *reinterpret_cast<const float4*>(cur + DIMP + r4);
        const float4 g4 = *reinterpret_cast<const float4*>(cur + 2 * DIMP + r4);
        const float kv[4] = {k4.x, k4.y, k4.z, k4.w}, qv[4] = {q4.x, q4.y, q4.z, q4.w}, gv[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = r4 + e;
          kk[r] = kv[e];
          s[r] *= gv[e];
          ak[r & 1] = fmaf(s[r], kv[e], ak[r & 1]);
          aq[r & 1] = fmaf(s[r], qv[e], aq[r & 1]);
          akq[r & 1] = fmaf(kv[e], qv[e], akq[r & 1]);
        }
      }
      float dot = ak[0] + ak[1], sq = aq[0] + aq[1], kq = akq[0] + akq[1];
#pragma unroll
      for (int o = WCOLS; o < 32; o <<= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        kq += __shfl_xor_sync(0xffffffffu, kq, o);
      }
      const float u = a.plain ? vj : bt * (vj - dot);
      const float out = fmaf(u, kq, sq);
#pragma unroll
      for (int r = 0; r < ROWS; ++r) s[r] = fmaf(kk[r], u, s[r]);
      if (active && part == 0) a.out[(size_t)(t0 + tok) * a.heads * a.vdim + (size_t)head * a.vdim + col] = out;
    }
    __syncthreads();             // the chunk is read: its buffer may take the chunk after the next
  }
  if (active) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int i = part * ROWS + r;
      if (i < dim) S[(size_t)i * a.vdim + col] = s[r];
    }
  }
}

template <int ROWS, int SPLIT>
int launch_recurrence_reg(const RecurArgs& a, int n_seqs, cudaStream_t stream) {
  constexpr int DIMP = (ROWS + 4) * SPLIT, BCOLS = (32 / SPLIT) * (kRecurThreads / 32);
  const size_t smem = (size_t)2 * kRecurTokens * (3 * DIMP + (BCOLS + 4) / 4 * 4) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_recurrence_reg_kernel<ROWS, SPLIT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((a.vdim + BCOLS - 1) / BCOLS, a.heads, n_seqs);
  delta_recurrence_reg_kernel<ROWS, SPLIT><<<grid, kRecurThreads, smem, stream>>>(a);
  return HB_OK;
}

// Any dim: the block's columns of S in shared memory, [dim][blockDim.x].
__global__ void delta_recurrence_smem_kernel(const RecurArgs a) {
  extern __shared__ float smem[];
  const int dim = a.dim, cols = blockDim.x;
  float* stage0 = smem;                 // [2][3 * dim]
  float* sm = smem + 6 * (size_t)dim;   // [dim][cols]
  const int head = blockIdx.y, seq = blockIdx.z;
  const int col = blockIdx.x * cols + threadIdx.x;
  const bool active = col < a.vdim;
  const int kvhead = head / (a.heads / a.kvh);
  const int first = a.cu_seqlens[seq], last = a.cu_seqlens[seq + 1];
  if (first >= last) return;
  float* S = a.state + (size_t)a.slots[seq] * a.state_stride + (size_t)head * dim * a.vdim;
  float* mine = sm + threadIdx.x;
  for (int i = 0; i < dim; ++i) mine[(size_t)i * cols] = active ? S[(size_t)i * a.vdim + col] : 0.f;
  stage_token(a, first, head, kvhead, stage0, dim);
  __syncthreads();
  for (int t = first; t < last; ++t) {
    const float* cur = stage0 + (size_t)((t - first) & 1) * 3 * dim;
    if (t + 1 < last) stage_token(a, t + 1, head, kvhead, stage0 + (size_t)((t - first + 1) & 1) * 3 * dim, dim);
    const float vj = active ? a.v[(size_t)t * a.heads * a.vdim + (size_t)head * a.vdim + col] : 0.f;
    const float bt = a.plain ? 1.f : a.beta[(size_t)t * a.heads + head];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < dim; ++i) {
      const float si = mine[(size_t)i * cols] * cur[2 * dim + i];
      mine[(size_t)i * cols] = si;
      acc[i & 3] = fmaf(si, cur[i], acc[i & 3]);
    }
    const float u = a.plain ? vj : bt * (vj - ((acc[0] + acc[1]) + (acc[2] + acc[3])));
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < dim; ++i) {
      const float si = fmaf(cur[i], u, mine[(size_t)i * cols]);
      mine[(size_t)i * cols] = si;
      o[i & 3] = fmaf(si, cur[dim + i], o[i & 3]);
    }
    if (active) a.out[(size_t)t * a.heads * a.vdim + (size_t)head * a.vdim + col] = (o[0] + o[1]) + (o[2] + o[3]);
    __syncthreads();
  }
  if (active)
    for (int i = 0; i < dim; ++i) S[(size_t)i * a.vdim + col] = mine[(size_t)i * cols];
}

// One warp per (token, head).
template <typename T>
__global__ void delta_out_norm_kernel(const float* __restrict__ o, const void* __restrict__ gate, int gate_dtype,
                                      const T* __restrict__ w, float eps, T* __restrict__ out, long long rows,
                                      int vdim, int gate_silu, long long gate_stride, int heads) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* src = o + row * vdim;
  float ss = 0.f;
  for (int j = lane; j < vdim; j += 32) ss += src[j] * src[j];
  const float inv = 1.f / sqrtf(hb::warp_sum(ss) / (float)vdim + eps);
  for (int j = lane; j < vdim; j += 32) {
    const float gx = ldf(gate, gate_dtype, (size_t)(row / heads) * gate_stride + (size_t)(row % heads) * vdim + j);
    const float g = gate_silu ? gx * sigmoid1(gx) : sigmoid1(gx);
    out[row * vdim + j] = hb::from_f32<T>(src[j] * inv * hb::to_f32(w[j]) * g);
  }
}

// q, k [N, heads * dim], v [N, heads * vdim] from columns of proj; decay = exp(-softplus(-(z + b)) / tau).
__global__ void gla_prep_kernel(const void* __restrict__ proj, int proj_dtype, long long ld, int q_off, int k_off,
                                int v_off, const float* __restrict__ z, const float* __restrict__ bias, float inv_tau,
                                float q_scale, float* __restrict__ q, float* __restrict__ k, float* __restrict__ v,
                                float* __restrict__ decay, int qk_cols, int v_cols) {
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < qk_cols; c += blockDim.x) {
    q[t * qk_cols + c] = ldf(proj, proj_dtype, t * ld + q_off + c) * q_scale;
    k[t * qk_cols + c] = ldf(proj, proj_dtype, t * ld + k_off + c);
    const float x = -(z[t * qk_cols + c] + (bias ? bias[c] : 0.f));
    const float sp = x > 20.f ? x : log1pf(expf(x));        // -log sigmoid(z + b)
    decay[t * qk_cols + c] = expf(-sp * inv_tau);
  }
  for (int c = threadIdx.x; c < v_cols; c += blockDim.x) v[t * v_cols + c] = ldf(proj, proj_dtype, t * ld + v_off + c);
}

}  // namespace

extern "C" int hb_gla_prep(const void* proj, int proj_dtype, long long ld, int q_off, int k_off, int v_off,
                           const float* z, const float* bias, float tau, float q_scale, float* q, float* k, float* v,
                           float* decay, int n_tokens, int qk_cols, int v_cols, cudaStream_t stream) {
  if (!proj || !z || !q || !k || !v || !decay || n_tokens < 0 || qk_cols <= 0 || v_cols <= 0 || !(tau > 0.f))
    return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  gla_prep_kernel<<<n_tokens, 256, 0, stream>>>(proj, proj_dtype, ld, q_off, k_off, v_off, z, bias, 1.f / tau, q_scale,
                                                q, k, v, decay, qk_cols, v_cols);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_delta_prep(const void* proj, int proj_dtype, long long ld, int chan_off, int beta_off,
                             const float* taps, float* state, long long state_stride, long long conv_off,
                             const void* a_pre, int a_dtype, const float* dt_bias, const float* a_log,
                             const int* cu_seqlens, const int* seq_of_token, const int* slots, float* q, float* k,
                             float* v, float* beta, float* decay, int n_tokens, int heads, int kvh, int dim, int vdim,
                             int taps_n, int head_decay, cudaStream_t stream) {
  if (!proj || !taps || !state || !a_pre || !dt_bias || !a_log || !cu_seqlens || !seq_of_token || !slots || !q || !k ||
      !v || !beta || !decay)
    return HB_ERR_BAD_ARG;
  if (heads <= 0 || kvh <= 0 || heads % kvh || dim <= 0 || vdim <= 0 || taps_n < 1 || n_tokens < 0) return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int longest = dim > vdim ? dim : vdim;
  const int warps = 4;
  const size_t smem = (size_t)warps * longest * sizeof(float);
  if (smem > 48 * 1024) return HB_ERR_UNSUPPORTED;
  PrepArgs a;
  a.proj = proj; a.proj_dtype = proj_dtype; a.ld = ld; a.chan_off = chan_off; a.beta_off = beta_off; a.taps = taps;
  a.state = state; a.state_stride = state_stride; a.conv_off = conv_off; a.a_pre = a_pre; a.a_dtype = a_dtype;
  a.head_decay = head_decay;
  a.dt_bias = dt_bias; a.a_log = a_log; a.cu_seqlens = cu_seqlens; a.seq_of_token = seq_of_token; a.slots = slots;
  a.q = q; a.k = k; a.v = v; a.beta = beta; a.decay = decay;
  a.heads = heads; a.kvh = kvh; a.dim = dim; a.vdim = vdim; a.K = taps_n;
  const int units = 2 * kvh + heads;
  int per_token = (units + warps - 1) / warps;
  if (per_token > 64) per_token = 64;
  delta_prep_kernel<<<dim3(n_tokens, per_token), warps * 32, smem, stream>>>(a, longest);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_delta_conv_update(const void* proj, int proj_dtype, long long ld, int chan_off, float* state,
                                    long long state_stride, long long conv_off, const int* cu_seqlens,
                                    const int* slots, int n_seqs, int channels, int taps_n, cudaStream_t stream) {
  if (!proj || !state || !cu_seqlens || !slots || channels <= 0 || taps_n < 1 || n_seqs < 0) return HB_ERR_BAD_ARG;
  if (n_seqs == 0 || taps_n == 1) return HB_OK;
  int per = (channels + 127) / 128;
  if (per > 16) per = 16;
  delta_conv_update_kernel<<<dim3(n_seqs, per), 128, 0, stream>>>(proj, proj_dtype, ld, chan_off, state, state_stride,
                                                                  conv_off, cu_seqlens, slots, channels, taps_n);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_delta_recurrence(const float* q, const float* k, const float* v, const float* beta,
                                   const float* decay, float* state, long long state_stride, const int* cu_seqlens,
                                   const int* slots, float* out, int n_seqs, int heads, int kvh, int dim, int vdim,
                                   int variant, int single_tokens, int plain, cudaStream_t stream) {
  if (!q || !k || !v || (!beta && !plain) || !decay || !state || !cu_seqlens || !slots || !out) return HB_ERR_BAD_ARG;
  if (heads <= 0 || kvh <= 0 || heads % kvh || dim <= 0 || vdim <= 0 || n_seqs < 0) return HB_ERR_BAD_ARG;
  if (n_seqs == 0) return HB_OK;
  RecurArgs a;
  a.q = q; a.k = k; a.v = v; a.beta = beta; a.decay = decay; a.state = state; a.state_stride = state_stride;
  a.cu_seqlens = cu_seqlens; a.slots = slots; a.out = out; a.heads = heads; a.kvh = kvh; a.dim = dim; a.vdim = vdim;
  a.plain = plain ? 1 : 0;
  if (variant != 1 && variant != 0 && variant != 16 && variant != 32) return HB_ERR_BAD_ARG;
  if (variant != 1 && dim <= 256) {
    // How many rows of a column a lane holds (`variant`, 0: chosen here). A step of single tokens is bound by
    // moving the states: 32 rows a lane, the widest runs of a row per warp (8 requests x 16 heads of 128 x 128:
    // 32 us against 37 us). A portion is bound by the chain from token to token: 16 rows a lane (2,048 tokens:
    // 766 us against 953 us; 8 rows a lane gave 777 us and are not built).
    const int rows = variant ? variant : (single_tokens && dim <= 128 ? 32 : 16);
    int code = HB_ERR_UNSUPPORTED;
    if (rows == 32)
      code = dim <= 32 ? launch_recurrence_reg<32, 1>(a, n_seqs, stream)
           : dim <= 64 ? launch_recurrence_reg<32, 2>(a, n_seqs, stream)
           : dim <= 128 ? launch_recurrence_reg<32, 4>(a, n_seqs, stream)
                        : launch_recurrence_reg<32, 8>(a, n_seqs, stream);
    else
      code = dim <= 32 ? launch_recurrence_reg<16, 2>(a, n_seqs, stream)
           : dim <= 64 ? launch_recurrence_reg<16, 4>(a, n_seqs, stream)
           : dim <= 128 ? launch_recurrence_reg<16, 8>(a, n_seqs, stream)
                        : launch_recurrence_reg<16, 16>(a, n_seqs, stream);
    if (code != HB_OK) return code;
  } else {
    const int cols = vdim > 32 ? 64 : 32;
    dim3 grid((vdim + cols - 1) / cols, heads, n_seqs);
    const size_t smem = ((size_t)6 * dim + (size_t)dim * cols) * sizeof(float);
    if (smem > 200 * 1024) return HB_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(delta_recurrence_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    delta_recurrence_smem_kernel<<<grid, cols, smem, stream>>>(a);
  }
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_delta_out_norm(const float* o, const void* gate, int gate_dtype, const void* w, float eps, void* out,
                                 int dtype, long long rows, int vdim, int gate_silu, long long gate_stride, int heads,
                                 cudaStream_t stream) {
  if (!o || !gate || !w || !out || rows < 0 || vdim <= 0 || heads <= 0 || gate_stride < (long long)heads * vdim)
    return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  const int warps = 4;
  const long long blocks = (rows + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;
  if (dtype == HB_DTYPE_F32)
    delta_out_norm_kernel<float><<<(int)blocks, warps * 32, 0, stream>>>(o, gate, gate_dtype, (const float*)w, eps,
                                                                         (float*)out, rows, vdim, gate_silu,
                                                                         gate_stride, heads);
  else if (dtype == HB_DTYPE_BF16)
    delta_out_norm_kernel<__nv_bfloat16><<<(int)blocks, warps * 32, 0, stream>>>(
        o, gate, gate_dtype, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)out, rows, vdim, gate_silu, gate_stride, heads);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

// Kernels of layers that keep a state per request instead of (or beside) a cache of keys:
// the residual sum + LayerNorm over a weighted sum of terms, the paged key/value write of
// layers that rotate nothing, the sigmoid gate per head, the short causal convolution,
// the linear recurrence (gated delta rule and state-space duality) and the gated RMS norm.
//
// Conventions.  Everything between a layer's projections and its output projection is
// float32 here: inputs are float32 matrices with a row stride (views into a projection's
// output), state is float32, and only what feeds the next product is stored as T.
// A step's tokens are ordered by request: `token_seq[t]` (the batch row of token t) never
// decreases, so the tokens of row b are a range that a binary search finds; `seq_seat[b]`
// is the request's slot in every state tensor.  Nothing here reads host-side batch data,
// so captured decode steps replay these kernels for whatever seats they are given.
#include "common.cuh"

namespace distie {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }

// First index t in [0, n) with token_seq[t] >= row (n if none).
__device__ __forceinline__ int first_token_of(const int* __restrict__ token_seq, int n, int row) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (token_seq[mid] < row) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// ---------------------------------------------------------------------------
// residual += sum_j scale_j * term_j (float32, written back), then
//   out = (residual - mean) / sqrt(var + eps) * weight + bias,  var = mean((residual - mean)^2).
// With `rows_index` only the listed rows are normalised and the residual stays as it is.
// One block per output row; the summed row waits in shared memory between the passes.
// ---------------------------------------------------------------------------
constexpr int kMaxTerms = 24;
struct SumTerms {
  const float* ptr[kMaxTerms];
  float scale[kMaxTerms];
  int count;
};

template <typename T>
__global__ void add_layernorm_kernel(SumTerms terms, float* __restrict__ residual, const float* __restrict__ weight,
                                     const float* __restrict__ bias, T* __restrict__ out,
                                     const int* __restrict__ rows_index, int hidden, float eps) {
  extern __shared__ float row_cache[];
  __shared__ float scratch[32];
  const int out_row = blockIdx.x;
  const int row = rows_index ? rows_index[out_row] : out_row;
  float* res = residual + (size_t)row * hidden;
  const bool write_back = terms.count > 0 && rows_index == nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float add = 0.f;
    for (int j = 0; j < terms.count; ++j) add += terms.scale[j] * terms.ptr[j][(size_t)row * hidden + i];
    const float v = res[i] + add;
    if (write_back) res[i] = v;
    row_cache[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / (float)hidden;
  float sq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row_cache[i] - mean;
    sq += d * d;
  }
  const float var = block_sum(sq, scratch) / (float)hidden;
  const float inv = 1.f / sqrtf(var + eps);
  T* dst = out + (size_t)out_row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    dst[i] = from_float<T>((row_cache[i] - mean) * inv * weight[i] + bias[i]);
}

// ---------------------------------------------------------------------------
// Keys and values of the new tokens into their pages, unrotated; a value may have another size
// than a key.  One block per token.
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void kv_write_kernel(const TIn* __restrict__ k, int k_stride, const TIn* __restrict__ v, int v_stride,
                                const int* __restrict__ positions, const int* __restrict__ token_seq,
                                const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                                T* __restrict__ k_cache, T* __restrict__ v_cache, int num_kv_heads, int head_dim,
                                int value_dim, int page_size, int num_pages, int* __restrict__ error) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seat = seq_seat[token_seq[t]];
  const int column = pos / page_size;
  const int page = (pos >= 0 && column < table_width) ? block_table[(size_t)seat * table_width + column] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0 && error) atomicExch(error, 2);
    return;
  }
  const int slot = pos % page_size;
  for (int e = threadIdx.x; e < num_kv_heads * head_dim; e += blockDim.x) {
    const int h = e / head_dim, d = e % head_dim;
    k_cache[(((size_t)page * num_kv_heads + h) * page_size + slot) * head_dim + d] =
        from_float<T>(to_float(k[(size_t)t * k_stride + e]));
  }
  for (int e = threadIdx.x; e < num_kv_heads * value_dim; e += blockDim.x) {
    const int h = e / value_dim, d = e % value_dim;
    v_cache[(((size_t)page * num_kv_heads + h) * page_size + slot) * value_dim + d] =
        from_float<T>(to_float(v[(size_t)t * v_stride + e]));
  }
}

// x[t, h, :] *= sigmoid(logits[t, h]).
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const float* __restrict__ logits, int logit_stride, int num_heads,
                                 int dim, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / ((size_t)num_heads * dim);
    const int h = (int)((i / dim) % num_heads);
    x[i] = from_float<T>(to_float(x[i]) * sigmoid_f(logits[t * logit_stride + h]));
  }
}

// ---------------------------------------------------------------------------
// Short causal convolution over time, per channel and per request.
//   y[t, c] = act(bias[c] + sum_j w[c, taps-1-j] * x_in(t - j)),  j = 0 .. taps-1
// where x_in reaches back into the request's state (its last taps-1 inputs, oldest first) for
// tokens before this step's portion.  A second kernel then moves the state on.
// ---------------------------------------------------------------------------
constexpr int kMaxTaps = 16;

__global__ void short_conv_kernel(const float* __restrict__ x, int x_stride, const float* __restrict__ weight,
                                  const float* __restrict__ bias, const float* __restrict__ state,
                                  const int* __restrict__ token_seq, const int* __restrict__ seq_seat, int tokens,
                                  int channels, int taps, int silu, float* __restrict__ out) {
  __shared__ int sh_first, sh_seat;
  const int t = blockIdx.y;
  if (threadIdx.x == 0) {
    const int row = token_seq[t];
    sh_first = first_token_of(token_seq, tokens, row);
    sh_seat = seq_seat[row];
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int first = sh_first;
  const float* held = state ? state + (size_t)sh_seat * (taps - 1) * channels : nullptr;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int at = t - j;
    float v;
    if (at >= first) v = x[(size_t)at * x_stride + c];
    else v = held ? held[(size_t)(at - first + taps - 1) * channels + c] : 0.f;
    acc += weight[(size_t)c * taps + (taps - 1 - j)] * v;
  }
  out[(size_t)t * channels + c] = silu ? silu_f(acc) : acc;
}

__global__ void short_conv_state_kernel(const float* __restrict__ x, int x_stride, float* __restrict__ state,
                                        const int* __restrict__ token_seq, const int* __restrict__ seq_seat,
                                        int tokens, int channels, int taps) {
  __shared__ int sh_first, sh_end, sh_seat;
  const int row = blockIdx.y;
  if (threadIdx.x == 0) {
    sh_first = first_token_of(token_seq, tokens, row);
    sh_end = first_token_of(token_seq, tokens, row + 1);
    sh_seat = seq_seat[row];
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int first = sh_first, n = sh_end - sh_first;
  if (c >= channels || n <= 0) return;
  float* held = state + (size_t)sh_seat * (taps - 1) * channels;
  float next[kMaxTaps];
  for (int i = 0; i < taps - 1; ++i) {
    const int rel = n + i - (taps - 1);  // index among this step's tokens of the request, negative: still the old state
    next[i] = rel >= 0 ? x[(size_t)(first + rel) * x_stride + c] : held[(size_t)(i + n) * channels + c];
  }
  for (int i = 0; i < taps - 1; ++i) held[(size_t)i * channels + c] = next[i];
}

// ---------------------------------------------------------------------------
// Linear recurrence with a matrix state per head and request, float32, token by token:
//   S <- g S;  S <- S + k u^T;  o = S^T q (+ skip * v)
// The columns of S (one per value element) never meet, so a column belongs to a group of
// eight lanes that share its key_dim entries (lane l holds i = 4 l + 32 r + c), and a block
// of 128 threads owns 16 columns of one head of one request.  Tokens come in tiles of 16:
// the block stages q, k, the 16 columns of v and the per-token scalars in shared memory,
// then every group walks the tile without meeting the others.
//   kDelta: q, k unit vectors (q times key_dim^-1/2); g = exp(-exp(rate) softplus(decay + bias));
//           u = sigmoid(write) (v - S^T k) with the decayed S.
//   kSsd:   dt = softplus(write + bias); g = exp(-exp(rate) dt); u = dt v; read-out + skip * v.
// State layout: [seat, head, value_dim, key_dim] (S transposed: a column is contiguous).
// ---------------------------------------------------------------------------
constexpr int kRuleDelta = 0, kRuleSsd = 1;
constexpr int kScanThreads = 128, kScanColumns = 16, kScanTile = 16;

struct ScanArgs {
  const float *q, *k, *v, *decay, *write;
  int q_stride, k_stride, v_stride, decay_stride, write_stride;
  const float *rate, *bias, *skip;
  float* state;
  float* out;
  int out_stride;
  const int *token_seq, *seq_seat;
  int tokens, heads, groups, key_dim, value_dim;
};

template <int PER, int RULE>
__global__ void __launch_bounds__(kScanThreads) linear_recurrence_kernel(ScanArgs a) {
  constexpr int KD = 8 * PER;
  __shared__ __align__(16) float sq[kScanTile][KD];
  __shared__ __align__(16) float sk[kScanTile][KD];
  __shared__ float sv[kScanTile][kScanColumns];
  __shared__ float sg[kScanTile], su[kScanTile];
  __shared__ int sh_first, sh_end, sh_seat;
  const int row = blockIdx.x, head = blockIdx.y;
  const int tid = threadIdx.x, lane8 = tid & 7, col_local = tid >> 3;
  const int j = blockIdx.z * kScanColumns + col_local;
  const bool valid = j < a.value_dim;
  const int grp = head / (a.heads / a.groups);
  if (tid == 0) {
    sh_first = first_token_of(a.token_seq, a.tokens, row);
    sh_end = first_token_of(a.token_seq, a.tokens, row + 1);
    sh_seat = a.seq_seat[row];
  }
  __syncthreads();
  const int first = sh_first, end = sh_end;
  if (end <= first) return;
  float* column = a.state + (((size_t)sh_seat * a.heads + head) * a.value_dim + (valid ? j : 0)) * a.key_dim;
  float S[PER];
#pragma unroll
  for (int r = 0; r < PER / 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = 4 * lane8 + 32 * r + c;
      S[4 * r + c] = (valid && i < a.key_dim) ? column[i] : 0.f;
    }
  const float rate = expf(a.rate[head]);
  const float bias = a.bias ? a.bias[head] : 0.f;
  const float skip = (RULE == kRuleSsd && a.skip) ? a.skip[head] : 0.f;
  const float q_scale = rsqrtf((float)a.key_dim);

  for (int tile = first; tile < end; tile += kScanTile) {
    const int count = min(kScanTile, end - tile);
    __syncthreads();  // the tile before is done with the shared arrays
    for (int idx = tid; idx < kScanTile * KD; idx += kScanThreads) {
      const int tok = idx / KD, i = idx % KD;
      const bool live = tok < count && i < a.key_dim;
      const size_t t = tile + tok;
      sq[tok][i] = live ? a.q[t * a.q_stride + grp * a.key_dim + i] : 0.f;
      sk[tok][i] = live ? a.k[t * a.k_stride + grp * a.key_dim + i] : 0.f;
    }
    for (int idx = tid; idx < kScanTile * kScanColumns; idx += kScanThreads) {
      const int tok = idx / kScanColumns, cj = blockIdx.z * kScanColumns + idx % kScanColumns;
      sv[tok][idx % kScanColumns] =
          (tok < count && cj < a.value_dim) ? a.v[(size_t)(tile + tok) * a.v_stride + head * a.value_dim + cj] : 0.f;
    }
    if (tid < count) {
      const size_t t = tile + tid;
      const float w = a.write[t * a.write_stride + head];
      if (RULE == kRuleDelta) {
        sg[tid] = expf(-rate * softplus_f(a.decay[t * a.decay_stride + head] + bias));
        su[tid] = sigmoid_f(w);
      } else {
        const float dt = softplus_f(w + bias);
        sg[tid] = expf(-rate * dt);
        su[tid] = dt;
      }
    }
    __syncthreads();
    if (RULE == kRuleDelta) {  // unit vectors: a warp per token
      const int lane = tid & 31, warp = tid >> 5;
      for (int tok = warp; tok < count; tok += kScanThreads / 32) {
        float qq = 0.f, kk = 0.f;
        for (int i = lane; i < KD; i += 32) { qq += sq[tok][i] * sq[tok][i]; kk += sk[tok][i] * sk[tok][i]; }
        qq = warp_sum(qq);
        kk = warp_sum(kk);
        const float qs = q_scale / sqrtf(qq + 1e-6f), ks = 1.f / sqrtf(kk + 1e-6f);
        for (int i = lane; i < KD; i += 32) { sq[tok][i] *= qs; sk[tok][i] *= ks; }
      }
      __syncthreads();
    }
    for (int tok = 0; tok < count; ++tok) {
      float kk[PER], qq[PER];
#pragma unroll
      for (int r = 0; r < PER / 4; ++r) {
        const float4 kv = *reinterpret_cast<const float4*>(&sk[tok][4 * lane8 + 32 * r]);
        const float4 qv = *reinterpret_cast<const float4*>(&sq[tok][4 * lane8 + 32 * r]);
        kk[4 * r] = kv.x; kk[4 * r + 1] = kv.y; kk[4 * r + 2] = kv.z; kk[4 * r + 3] = kv.w;
        qq[4 * r] = qv.x; qq[4 * r + 1] = qv.y; qq[4 * r + 2] = qv.z; qq[4 * r + 3] = qv.w;
      }
      const float g = sg[tok], vj = sv[tok][col_local];
      float u;
      if (RULE == kRuleDelta) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < PER; ++e) dot += S[e] * kk[e];
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        u = su[tok] * (vj - g * dot);
      } else {
        u = su[tok] * vj;
      }
      float o = 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        S[e] = g * S[e] + kk[e] * u;
        o += S[e] * qq[e];
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      if (lane8 == 0 && valid) a.out[(size_t)(tile + tok) * a.out_stride + head * a.value_dim + j] = o + skip * vj;
    }
  }
  if (valid) {
#pragma unroll
    for (int r = 0; r < PER / 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = 4 * lane8 + 32 * r + c;
        if (i < a.key_dim) column[i] = S[4 * r + c];
      }
  }
}

template <int RULE>
static cudaError_t launch_scan(const ScanArgs& a, int num_seqs, cudaStream_t stream) {
  const dim3 grid(num_seqs, a.heads, (a.value_dim + kScanColumns - 1) / kScanColumns);
  if (a.key_dim <= 32) linear_recurrence_kernel<4, RULE><<<grid, kScanThreads, 0, stream>>>(a);
  else if (a.key_dim <= 64) linear_recurrence_kernel<8, RULE><<<grid, kScanThreads, 0, stream>>>(a);
  else if (a.key_dim <= 128) linear_recurrence_kernel<16, RULE><<<grid, kScanThreads, 0, stream>>>(a);
  else linear_recurrence_kernel<32, RULE><<<grid, kScanThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// RMS norm over groups of `group` neighbouring columns with a SiLU gate, a warp per (token, group):
//   gate_first: norm(x * silu(gate)) * weight;   else: norm(x) * weight * silu(gate).
// weight has `weight_len` elements and repeats along the row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ x, int x_stride, const float* __restrict__ gate,
                                     int gate_stride, const float* __restrict__ weight, int weight_len, T* __restrict__ out,
                                     int out_stride, int tokens, int groups, int group, float eps, int gate_first) {
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)tokens * groups) return;
  const int t = (int)(unit / groups), part = (int)(unit % groups);
  const float* xr = x + (size_t)t * x_stride + (size_t)part * group;
  const float* gr = gate + (size_t)t * gate_stride + (size_t)part * group;
  float sq = 0.f;
  for (int i = lane; i < group; i += 32) {
    const float v = gate_first ? xr[i] * silu_f(gr[i]) : xr[i];
    sq += v * v;
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / (float)group + eps);
  T* dst = out + (size_t)t * out_stride + (size_t)part * group;
  for (int i = lane; i < group; i += 32) {
    const float s = silu_f(gr[i]);
    const float w = weight[(part * group + i) % weight_len];
    dst[i] = from_float<T>(gate_first ? xr[i] * s * inv * w : xr[i] * inv * w * s);
  }
}

}  // namespace distie

using namespace distie;

extern "C" int distie_add_layernorm(const float* const* term_ptrs, const float* term_scales, int num_terms,
                                    float* residual, const float* weight, const float* bias, void* out,
                                    const int* rows_index, int rows, int hidden, float eps, int dtype,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden < 1 || num_terms < 0 || num_terms > kMaxTerms) return DISTIE_ERR_ARG;
  SumTerms terms;
  terms.count = num_terms;
  for (int j = 0; j < num_terms; ++j) { terms.ptr[j] = term_ptrs[j]; terms.scale[j] = term_scales[j]; }
  const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  const size_t shared = (size_t)hidden * sizeof(float);
  if (shared > 200 * 1024) return DISTIE_ERR_UNSUPPORTED;
  if (dtype == DISTIE_BF16) {
    if (shared > 48 * 1024)
      cudaFuncSetAttribute(add_layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    add_layernorm_kernel<<<rows, threads, shared, stream>>>(terms, residual, weight, bias, (__nv_bfloat16*)out,
                                                            rows_index, hidden, eps);
  } else if (dtype == DISTIE_F32) {
    if (shared > 48 * 1024)
      cudaFuncSetAttribute(add_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    add_layernorm_kernel<<<rows, threads, shared, stream>>>(terms, residual, weight, bias, (float*)out, rows_index,
                                                            hidden, eps);
  } else {
    return DISTIE_ERR_UNSUPPORTED;
  }
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_kv_write(const void* k, int k_stride, const void* v, int v_stride, int in_dtype,
                               const int* positions, const int* token_seq, const int* seq_seat, const int* block_table,
                               int table_width, void* k_cache, void* v_cache, int tokens, int num_kv_heads, int head_dim,
                               int value_dim, int page_size, int num_pages, int dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_kv_heads < 1 || head_dim < 1 || value_dim < 1 || page_size < 1 || table_width < 1) return DISTIE_ERR_ARG;
  const int threads = 128;
#define DISTIE_KV_WRITE(TIN, T)                                                                                      \
  kv_write_kernel<<<tokens, threads, 0, stream>>>((const TIN*)k, k_stride, (const TIN*)v, v_stride, positions,        \
                                                  token_seq, seq_seat, block_table, table_width, (T*)k_cache,         \
                                                  (T*)v_cache, num_kv_heads, head_dim, value_dim, page_size,          \
                                                  num_pages, error)
  if (in_dtype == DISTIE_F32 && dtype == DISTIE_F32) DISTIE_KV_WRITE(float, float);
  else if (in_dtype == DISTIE_F32 && dtype == DISTIE_BF16) DISTIE_KV_WRITE(float, __nv_bfloat16);
  else if (in_dtype == DISTIE_BF16 && dtype == DISTIE_BF16) DISTIE_KV_WRITE(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == DISTIE_BF16 && dtype == DISTIE_F32) DISTIE_KV_WRITE(__nv_bfloat16, float);
  else return DISTIE_ERR_UNSUPPORTED;
#undef DISTIE_KV_WRITE
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_head_gate(void* x, const float* logits, int logit_stride, int tokens, int num_heads, int dim,
                                int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || dim < 1) return DISTIE_ERR_ARG;
  const size_t total = (size_t)tokens * num_heads * dim;
  const int threads = 256;
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == DISTIE_BF16)
    head_gate_kernel<<<blocks, threads, 0, stream>>>((__nv_bfloat16*)x, logits, logit_stride, num_heads, dim, total);
  else if (dtype == DISTIE_F32)
    head_gate_kernel<<<blocks, threads, 0, stream>>>((float*)x, logits, logit_stride, num_heads, dim, total);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// state may be null only when taps == 1.
extern "C" int distie_short_conv(const float* x, int x_stride, const float* weight, const float* bias, float* state,
                                 const int* token_seq, const int* seq_seat, int tokens, int num_seqs, int channels,
                                 int taps, int silu, float* out, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels < 1 || taps < 1 || num_seqs < 1) return DISTIE_ERR_ARG;
  if (taps > kMaxTaps) return DISTIE_ERR_UNSUPPORTED;
  if (taps > 1 && state == nullptr) return DISTIE_ERR_ARG;
  const int threads = 128;
  const dim3 grid((channels + threads - 1) / threads, tokens);
  short_conv_kernel<<<grid, threads, 0, stream>>>(x, x_stride, weight, bias, state, token_seq, seq_seat, tokens,
                                                  channels, taps, silu, out);
  DISTIE_LAUNCH_CHECK();
  if (taps > 1) {
    const dim3 grid_state((channels + threads - 1) / threads, num_seqs);
    short_conv_state_kernel<<<grid_state, threads, 0, stream>>>(x, x_stride, state, token_seq, seq_seat, tokens,
                                                                channels, taps);
    DISTIE_LAUNCH_CHECK();
  }
  return 0;
}

extern "C" int distie_linear_recurrence(int rule, const float* q, int q_stride, const float* k, int k_stride,
                                        const float* v, int v_stride, const float* decay, int decay_stride,
                                        const float* write, int write_stride, const float* rate, const float* bias,
                                        const float* skip, float* state, float* out, int out_stride,
                                        const int* token_seq, const int* seq_seat, int tokens, int num_seqs, int heads,
                                        int groups, int key_dim, int value_dim, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || key_dim < 1 || value_dim < 1 || num_seqs < 1 || heads > 65535)
    return DISTIE_ERR_ARG;
  if (key_dim > 256 || (value_dim + kScanColumns - 1) / kScanColumns > 65535) return DISTIE_ERR_UNSUPPORTED;
  if (rate == nullptr || state == nullptr || (rule == kRuleDelta && decay == nullptr)) return DISTIE_ERR_ARG;
  ScanArgs a;
  a.q = q; a.k = k; a.v = v; a.decay = decay; a.write = write;
  a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride; a.decay_stride = decay_stride;
  a.write_stride = write_stride;
  a.rate = rate; a.bias = bias; a.skip = skip; a.state = state; a.out = out; a.out_stride = out_stride;
  a.token_seq = token_seq; a.seq_seat = seq_seat;
  a.tokens = tokens; a.heads = heads; a.groups = groups; a.key_dim = key_dim; a.value_dim = value_dim;
  cudaError_t err;
  if (rule == kRuleDelta) err = launch_scan<kRuleDelta>(a, num_seqs, stream);
  else if (rule == kRuleSsd) err = launch_scan<kRuleSsd>(a, num_seqs, stream);
  else return DISTIE_ERR_ARG;
  return err == cudaSuccess ? 0 : (int)err;
}

extern "C" int distie_gated_rmsnorm(const float* x, int x_stride, const float* gate, int gate_stride,
                                    const float* weight, int weight_len, void* out, int out_stride, int tokens, int n,
                                    int group, float eps, int gate_first, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n < 1 || group < 1 || n % group || weight_len < 1) return DISTIE_ERR_ARG;
  const int groups = n / group, warps = 4;
  const long long units = (long long)tokens * groups;
  const unsigned blocks = (unsigned)((units + warps - 1) / warps);
  if (dtype == DISTIE_BF16)
    gated_rmsnorm_kernel<<<blocks, warps * 32, 0, stream>>>(x, x_stride, gate, gate_stride, weight, weight_len,
                                                            (__nv_bfloat16*)out, out_stride, tokens, groups, group, eps,
                                                            gate_first);
  else if (dtype == DISTIE_F32)
    gated_rmsnorm_kernel<<<blocks, warps * 32, 0, stream>>>(x, x_stride, gate, gate_stride, weight, weight_len,
                                                            (float*)out, out_stride, tokens, groups, group, eps,
                                                            gate_first);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

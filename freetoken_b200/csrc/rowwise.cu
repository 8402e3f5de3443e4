// Row-wise kernels of mixers that keep ONE tensor per token in the cache (keys
// that are also the values, or a latent vector), of plain two-matrix
// feed-forwards, and of heads and embeddings with a norm or a cap of their own.
//
// All arithmetic is float32 whatever the storage type; a block (or a thread)
// owns one token, so a token's result does not depend on what else is in the
// launch.
//
//   embed_norm      r[t,:] = rms(E[id_t,:]) * g          (gather + RMS norm in one pass)
//   key_store       q_out[t,h,:] = q[t,h,:] * (1 + coef * ln(floor((p_t + 1) / every) + 1))
//                   k[t,g,:] -> (optionally rms(k) * w, per key head) -> page of p_t
//   gate_heads      o[t,h,:] *= sigmoid(z[t,h])
//   activation      y = f(x): relu(x)^2, tanh-GELU, SiLU
//   softcap         y = cap * tanh(y / cap)
#include "common.cuh"

namespace ft {

// ------------------------------------------------------------- embed + norm
template <typename WT>
__global__ void __launch_bounds__(256)
embed_norm_kernel(const int* __restrict__ ids, const WT* __restrict__ table,
                  const float* __restrict__ weight, float* __restrict__ residual, int H, int vocab,
                  float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // validated on the host; never index outside the table
  const WT* row = table + (size_t)id * H;
  float* out = residual + (size_t)t * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = to_float(row[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_float(row[i]) * inv * weight[i];
}

// ---------------------------------------------------------------- key store
struct KeyStoreArgs {
  const void* src;        // [T, ld]: a projection's rows; queries at q_off, keys at k_off
  void* q_out;            // [T, nq*dq] or nullptr (queries are left where they are)
  void* pages;            // [pages, nkv, P, dk] or nullptr (a stop that reads another stop's cache)
  const float* k_weight;  // [dk] or nullptr: RMS norm of every key head's row, times this
  const int* token_pos;   // [T]
  const int* token_seg;   // [T]
  const int* block_table; // [S, table_width]
  long long ld, page_stride;
  int q_off, k_off, nq, dq, nkv, dk, P, table_width, every;
  float coef, eps;
};

template <typename AT>
__global__ void __launch_bounds__(128) key_store_kernel(KeyStoreArgs a) {
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const AT* row = (const AT*)a.src + (size_t)t * a.ld;
  const int pos = a.token_pos[t];
  if (a.q_out) {
    // the temperature is a function of the position alone, in float32
    float temp = 1.f;
    if (a.coef != 0.f) temp = 1.f + a.coef * logf((float)((pos + 1) / a.every) + 1.f);
    AT* qo = (AT*)a.q_out + (size_t)t * a.nq * a.dq;
    const AT* q = row + a.q_off;
    for (int i = threadIdx.x; i < a.nq * a.dq; i += blockDim.x) qo[i] = from_float<AT>(to_float(q[i]) * temp);
  }
  if (!a.pages) return;
  const int page = a.block_table[(size_t)a.token_seg[t] * a.table_width + pos / a.P];
  AT* dst = (AT*)a.pages + (size_t)page * a.page_stride + (size_t)(pos % a.P) * a.dk;
  for (int g = warp; g < a.nkv; g += nwarps) {
    const AT* k = row + a.k_off + (size_t)g * a.dk;
    AT* kd = dst + (size_t)g * a.P * a.dk;
    if (a.k_weight) {
      float ss = 0.f;
      for (int i = lane; i < a.dk; i += 32) {
        const float v = to_float(k[i]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)a.dk + a.eps);
      for (int i = lane; i < a.dk; i += 32) kd[i] = from_float<AT>(to_float(k[i]) * inv * a.k_weight[i]);
    } else {
      for (int i = lane; i < a.dk; i += 32) kd[i] = k[i];
    }
  }
}

// ------------------------------------------------------------------- gates
// o[t, h, 0..d) *= sigmoid(z[t*ldz + h])
template <typename AT>
__global__ void __launch_bounds__(256)
gate_heads_kernel(AT* __restrict__ o, const AT* __restrict__ z, long long ldz, int heads, int d, long long n) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long th = i / d;
  const long long t = th / heads;
  const int h = (int)(th - t * heads);
  const float zz = to_float(z[t * ldz + h]);
  const float g = 1.f / (1.f + expf(-zz));
  o[i] = from_float<AT>(to_float(o[i]) * g);
}

// -------------------------------------------------------------- activation
__device__ __forceinline__ float act_apply(float x, int kind) {
  switch (kind) {
    case 0: { const float r = fmaxf(x, 0.f); return r * r; }                     // relu squared
    case 1: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));  // tanh-GELU
    default: return x / (1.f + expf(-x));                                         // SiLU
  }
}

template <typename AT>
__global__ void __launch_bounds__(256) activation_kernel(AT* __restrict__ x, long long n, int kind) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = from_float<AT>(act_apply(to_float(x[i]), kind));
}

// 8 bfloat16 values a thread
__global__ void __launch_bounds__(256) activation_bf16x8_kernel(uint4* __restrict__ x, long long n8, int kind) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  uint4 raw = x[i];
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __bfloat1622float2(p[j]);
    p[j] = __floats2bfloat162_rn(act_apply(v.x, kind), act_apply(v.y, kind));
  }
  x[i] = raw;
}

// ------------------------------------------------------------------ softcap
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ x, long long n, float cap) {
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace ft

using namespace ft;

extern "C" {

int ft_embed_norm(const int* ids, const void* table, int table_dtype, const float* weight, float* residual,
                  int T, int H, int vocab, float eps, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  FT_DISPATCH(table_dtype, WT,
              launch_pdl(embed_norm_kernel<WT>, dim3(T), dim3(256), 0, stream, ids, (const WT*)table, weight,
                         residual, H, vocab, eps));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_key_store(const void* src, void* q_out, void* pages, const float* k_weight, const int* token_pos,
                 const int* token_seg, const int* block_table, long long ld, long long page_stride,
                 int q_off, int k_off, int nq, int dq, int nkv, int dk, int P, int table_width, int every,
                 float coef, float eps, int dtype, int T, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (nkv <= 0 || dk <= 0 || P <= 0 || (coef != 0.f && every <= 0)) return FT_ERR_SHAPE;
  KeyStoreArgs a{src, q_out, pages, k_weight, token_pos, token_seg, block_table, ld, page_stride,
                 q_off, k_off, nq, dq, nkv, dk, P, table_width, every, coef, eps};
  FT_DISPATCH(dtype, AT, launch_pdl(key_store_kernel<AT>, dim3(T), dim3(128), 0, stream, a));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_gate_heads(void* o, const void* z, long long ldz, int heads, int d, int dtype, int T, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  const long long n = (long long)T * heads * d;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  FT_DISPATCH(dtype, AT,
              launch_pdl(gate_heads_kernel<AT>, dim3(blocks), dim3(256), 0, stream, (AT*)o, (const AT*)z, ldz,
                         heads, d, n));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_activation(void* x, long long n, int kind, int dtype, cudaStream_t stream) {
  if (n <= 0) return FT_OK;
  if (kind < 0 || kind > 2) return FT_ERR_SHAPE;
  if (dtype == FT_DTYPE_BF16 && !(n & 7) && !((uintptr_t)x & 15)) {
    const long long n8 = n >> 3;
    launch_pdl(activation_bf16x8_kernel, dim3((unsigned)((n8 + 255) / 256)), dim3(256), 0, stream, (uint4*)x, n8,
               kind);
    FT_LAUNCH_CHECK();
    return FT_OK;
  }
  FT_DISPATCH(dtype, AT,
              launch_pdl(activation_kernel<AT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (AT*)x, n,
                         kind));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return FT_OK;
  if (!(cap > 0.f)) return FT_ERR_SHAPE;
  launch_pdl(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap);
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"

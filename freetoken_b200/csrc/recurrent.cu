// Mixers that carry a state of fixed size from token to token: a short causal
// convolution over time, a selective state space with one decay per head
// (Mamba-2's recurrence), the gated delta rule, and the gated norm behind both.
//
// Everything that enters a recurrence is float32 whatever the activation type:
// step sizes (softplus), decays (exp), gates (sigmoid), unit norms and the state
// itself.  A request's tokens are taken in order; a segment of a step continues
// from the state its request's slot holds and leaves the state there.  A token's
// result depends on its own request alone: on nothing else in the launch, and on
// how the request was cut into steps only through float32 rounding (it is not:
// every token performs the same operations in the same order whatever the cut).
//
//   conv_silu        y[t,c] = silu(b_c + sum_j w[c,j] u[t-(taps-1)+j, c]); the last
//                    taps-1 inputs of a request live in its state slot
//   ssd_scan         S <- exp(-exp(A) dt) S + dt B x^T ; y = S^T C + D x       (S: N x P per head)
//   delta_scan       S <- g S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q   (S: D x P per head)
//   gated_norm       rms over groups of a row, a gate silu(z) before or after it
//
// State layout per head: [N or D][P] float32, P contiguous.  A warp owns WC
// columns of a head's state and its lanes split the rows, so a column's dot
// products are one warp reduction; a block's four warps share the tokens of a
// chunk, which all threads stage into shared memory together.
#include "common.cuh"

namespace ft {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// Sums V values per lane over the warp with V - 1 + log2(32 / V) shuffles: at every step a lane
// hands half of its values to the lane `mask` away and adds what it gets to the half it keeps.
// Afterwards v[0] of lane l is the warp's total of value  l >> (5 - log2 V).
template <int V>
__device__ __forceinline__ void warp_sum_multi(float (&v)[V]) {
  const int lane = threadIdx.x & 31;
  int mask = 16;
#pragma unroll
  for (int w = V / 2; w >= 1; w >>= 1) {
    const bool upper = lane & mask;
#pragma unroll
    for (int i = 0; i < w; ++i) {
      const float send = upper ? v[i] : v[i + w];
      const float keep = upper ? v[i + w] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
    mask >>= 1;
  }
  for (; mask >= 1; mask >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], mask);
}
template <int V> struct Log2 { static constexpr int value = 1 + Log2<V / 2>::value; };
template <> struct Log2<1> { static constexpr int value = 0; };

// ------------------------------------------------------------ short convolution
struct ConvArgs {
  const void* x;        // [T, ldx]: channel c of token t at x[t * ldx + c]
  void* out;            // [T, ldo]
  const float* w;       // [C, taps]; the last column weighs the current token
  const float* bias;    // [C] or nullptr
  float* state;         // slot s: state + s * slot_stride, [taps - 1][C], oldest input first
  const int* token_seg; // [T]
  const int* seg_slot;  // [S]
  const int* seg_q_start;  // [S + 1]
  long long ldx, ldo, slot_stride;
  int C, taps;
};

template <typename AT>
__global__ void __launch_bounds__(128) conv_silu_kernel(ConvArgs a) {
  pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int seg = a.token_seg[t];
  const int q0 = a.seg_q_start[seg];
  const int r = t - q0, K = a.taps - 1;
  const float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride;
  const AT* x = (const AT*)a.x;
  float acc = 0.f;
  for (int j = 0; j <= K; ++j) {
    const int s = r - K + j;
    const float v = s >= 0 ? to_float(x[(size_t)(q0 + s) * a.ldx + c]) : st[(size_t)(K + s) * a.C + c];
    acc = fmaf(a.w[(size_t)c * a.taps + j], v, acc);
  }
  if (a.bias) acc += a.bias[c];
  ((AT*)a.out)[(size_t)t * a.ldo + c] = from_float<AT>(silu_f(acc));
}

// After the convolution has read it: the slot keeps the last taps-1 inputs of (what it held ++
// the segment's inputs).  Ascending i reads entries at or above the one it writes.
template <typename AT>
__global__ void __launch_bounds__(128) conv_state_kernel(ConvArgs a) {
  pdl_wait();
  const int seg = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const int q0 = a.seg_q_start[seg], n = a.seg_q_start[seg + 1] - q0, K = a.taps - 1;
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride;
  const AT* x = (const AT*)a.x;
  for (int i = 0; i < K; ++i) {
    const int src = n + i;
    st[(size_t)i * a.C + c] = src < K ? st[(size_t)src * a.C + c] : to_float(x[(size_t)(q0 + src - K) * a.ldx + c]);
  }
}

// -------------------------------------------------------- selective state space
constexpr int SCAN_WARPS = 4;
constexpr int SCAN_WC = 8;                       // state columns a warp owns
constexpr int SCAN_COLS = SCAN_WARPS * SCAN_WC;  // ... a block owns
constexpr int SCAN_CHUNK = 16;                   // tokens staged in shared memory at a time

struct SsdArgs {
  const void* xbc;      // [T, ld]: x (heads * P) | B (G * N) | C (G * N), after convolution and silu
  const void* dt;       // [T, ld_dt]: the step size's projection, head h at column h
  const float* dt_bias; // [heads]
  const float* A_log;   // [heads]
  const float* D;       // [heads]
  float* state;         // slot s: state + s * slot_stride, [heads][N][P]
  float* y;             // [T, heads * P] float32
  const int* seg_slot;
  const int* seg_q_start;
  long long ld, ld_dt, slot_stride;
  int heads, P, N, G;
};

// NPL: state rows a lane holds (N <= 32 * NPL)
template <typename AT, int NPL>
__global__ void __launch_bounds__(SCAN_WARPS * 32) ssd_scan_kernel(SsdArgs a) {
  extern __shared__ float sm[];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y, seg = blockIdx.z;
  const int N = a.N, P = a.P;
  const int g = head / (a.heads / a.G);
  const int inner = a.heads * P;
  const int col0 = blockIdx.x * SCAN_COLS;           // first column of the block
  const int j0 = col0 + warp * SCAN_WC;              // first column of the warp
  float* Bs = sm;                                     // [CHUNK][N]
  float* Cs = Bs + SCAN_CHUNK * N;                    // [CHUNK][N]
  float* xs = Cs + SCAN_CHUNK * N;                    // [CHUNK][SCAN_COLS]
  float* dts = xs + SCAN_CHUNK * SCAN_COLS;           // [CHUNK] step size
  float* das = dts + SCAN_CHUNK;                      // [CHUNK] decay
  const int q0 = a.seg_q_start[seg], q1 = a.seg_q_start[seg + 1];
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + (size_t)head * N * P;
  const float rate = -expf(a.A_log[head]), bias = a.dt_bias[head], skip = a.D[head];

  float S[NPL][SCAN_WC];
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
#pragma unroll
    for (int c = 0; c < SCAN_WC; ++c)
      S[e][c] = (n < N && j0 + c < P) ? st[(size_t)n * P + j0 + c] : 0.f;
  }
  const AT* xbc = (const AT*)a.xbc;
  const AT* dt = (const AT*)a.dt;
  for (int t0 = q0; t0 < q1; t0 += SCAN_CHUNK) {
    const int nt = min(SCAN_CHUNK, q1 - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
      const int tt = i / N, n = i % N;
      const AT* row = xbc + (size_t)(t0 + tt) * a.ld + inner + (size_t)g * N + n;
      Bs[tt * N + n] = to_float(row[0]);
      Cs[tt * N + n] = to_float(row[(size_t)a.G * N]);
    }
    for (int i = threadIdx.x; i < nt * SCAN_COLS; i += blockDim.x) {
      const int tt = i / SCAN_COLS, c = i % SCAN_COLS;
      xs[i] = col0 + c < P ? to_float(xbc[(size_t)(t0 + tt) * a.ld + (size_t)head * P + col0 + c]) : 0.f;
    }
    if (threadIdx.x < nt) {
      const float step = softplus_f(to_float(dt[(size_t)(t0 + threadIdx.x) * a.ld_dt + head]) + bias);
      dts[threadIdx.x] = step;
      das[threadIdx.x] = expf(rate * step);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float step = dts[tt], decay = das[tt];
      float Bv[NPL], Cv[NPL];
#pragma unroll
      for (int e = 0; e < NPL; ++e) {
        const int n = lane + 32 * e;
        Bv[e] = n < N ? Bs[tt * N + n] : 0.f;
        Cv[e] = n < N ? Cs[tt * N + n] : 0.f;
      }
      float part[SCAN_WC];
#pragma unroll
      for (int c = 0; c < SCAN_WC; ++c) {
        const float xv = xs[tt * SCAN_COLS + warp * SCAN_WC + c];
        const float in = step * xv;
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < NPL; ++e) {
          S[e][c] = fmaf(decay, S[e][c], in * Bv[e]);
          acc = fmaf(S[e][c], Cv[e], acc);
        }
        part[c] = acc;
      }
      warp_sum_multi<SCAN_WC>(part);
      const int c = lane >> (5 - Log2<SCAN_WC>::value);
      if ((lane & ((32 / SCAN_WC) - 1)) == 0 && j0 + c < P)
        a.y[(size_t)(t0 + tt) * inner + (size_t)head * P + j0 + c] =
            part[0] + skip * xs[tt * SCAN_COLS + warp * SCAN_WC + c];
    }
  }
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
#pragma unroll
    for (int c = 0; c < SCAN_WC; ++c)
      if (n < N && j0 + c < P) st[(size_t)n * P + j0 + c] = S[e][c];
  }
}

// ------------------------------------------------------------- gated delta rule
struct DeltaArgs {
  const void* qkv;      // [T, ld]: q (G * D) | k (G * D) | v (heads * P), after convolution and silu
  const void* beta;     // [T, ld_gate]: the write strength's projection, head h at column h
  const void* decay;    // [T, ld_gate]: the decay's projection, head h at column h
  const float* dt_bias; // [heads]
  const float* A_log;   // [heads]
  float* state;         // slot s: state + s * slot_stride, [heads][D][P]
  float* o;             // [T, heads * P] float32
  const int* seg_slot;
  const int* seg_q_start;
  long long ld, ld_gate, slot_stride;
  int heads, P, D, G;
  float unit_eps, q_scale;
};

template <typename AT, int NPL>
__global__ void __launch_bounds__(SCAN_WARPS * 32) delta_scan_kernel(DeltaArgs a) {
  extern __shared__ float sm[];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y, seg = blockIdx.z;
  const int D = a.D, P = a.P;
  const int g = head / (a.heads / a.G);
  const int col0 = blockIdx.x * SCAN_COLS;
  const int j0 = col0 + warp * SCAN_WC;
  const int width = a.heads * P;
  float* qs = sm;                                     // [CHUNK][D] unit q times q_scale
  float* ks = qs + SCAN_CHUNK * D;                    // [CHUNK][D] unit k
  float* vs = ks + SCAN_CHUNK * D;                    // [CHUNK][SCAN_COLS]
  float* bs = vs + SCAN_CHUNK * SCAN_COLS;            // [CHUNK] beta
  float* gs = bs + SCAN_CHUNK;                        // [CHUNK] decay
  float* kqs = gs + SCAN_CHUNK;                       // [CHUNK] k . q
  const int q0 = a.seg_q_start[seg], q1 = a.seg_q_start[seg + 1];
  float* st = a.state + (size_t)a.seg_slot[seg] * a.slot_stride + (size_t)head * D * P;
  const float rate = -expf(a.A_log[head]), bias = a.dt_bias[head];

  float S[NPL][SCAN_WC];
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
#pragma unroll
    for (int c = 0; c < SCAN_WC; ++c)
      S[e][c] = (n < D && j0 + c < P) ? st[(size_t)n * P + j0 + c] : 0.f;
  }
  const AT* qkv = (const AT*)a.qkv;
  for (int t0 = q0; t0 < q1; t0 += SCAN_CHUNK) {
    const int nt = min(SCAN_CHUNK, q1 - t0);
    __syncthreads();
    // a warp makes unit vectors of the q and k rows of every fourth token
    for (int tt = warp; tt < nt; tt += SCAN_WARPS) {
      const AT* qrow = qkv + (size_t)(t0 + tt) * a.ld + (size_t)g * D;
      const AT* krow = qrow + (size_t)a.G * D;
      float qv[NPL], kv[NPL], sq = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < NPL; ++e) {
        const int n = lane + 32 * e;
        qv[e] = n < D ? to_float(qrow[n]) : 0.f;
        kv[e] = n < D ? to_float(krow[n]) : 0.f;
        sq = fmaf(qv[e], qv[e], sq);
        sk = fmaf(kv[e], kv[e], sk);
      }
      const float iq = a.q_scale / sqrtf(warp_sum(sq) + a.unit_eps);
      const float ik = 1.f / sqrtf(warp_sum(sk) + a.unit_eps);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < NPL; ++e) {
        const int n = lane + 32 * e;
        qv[e] *= iq;
        kv[e] *= ik;
        dot = fmaf(qv[e], kv[e], dot);
        if (n < D) {
          qs[tt * D + n] = qv[e];
          ks[tt * D + n] = kv[e];
        }
      }
      dot = warp_sum(dot);
      if (lane == 0) {
        kqs[tt] = dot;
        const size_t at = (size_t)(t0 + tt) * a.ld_gate + head;
        bs[tt] = 1.f / (1.f + expf(-to_float(((const AT*)a.beta)[at])));
        gs[tt] = expf(rate * softplus_f(to_float(((const AT*)a.decay)[at]) + bias));
      }
    }
    for (int i = threadIdx.x; i < nt * SCAN_COLS; i += blockDim.x) {
      const int tt = i / SCAN_COLS, c = i % SCAN_COLS;
      vs[i] = col0 + c < P
                  ? to_float(qkv[(size_t)(t0 + tt) * a.ld + 2 * (size_t)a.G * D + (size_t)head * P + col0 + c])
                  : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float beta = bs[tt], decay = gs[tt], kq = kqs[tt];
      float qv[NPL], kv[NPL];
#pragma unroll
      for (int e = 0; e < NPL; ++e) {
        const int n = lane + 32 * e;
        qv[e] = n < D ? qs[tt * D + n] : 0.f;
        kv[e] = n < D ? ks[tt * D + n] : 0.f;
      }
      // per column: a = S^T k and b = S^T q of the state before this token
      float red[2 * SCAN_WC];
#pragma unroll
      for (int c = 0; c < SCAN_WC; ++c) {
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int e = 0; e < NPL; ++e) {
          sa = fmaf(S[e][c], kv[e], sa);
          sb = fmaf(S[e][c], qv[e], sb);
        }
        red[c] = sa;
        red[SCAN_WC + c] = sb;
      }
      warp_sum_multi<2 * SCAN_WC>(red);
      // lane l holds the total of value l >> 1: even pairs of lanes a_c, the upper half b_c
      const float mine = red[0];
#pragma unroll
      for (int c = 0; c < SCAN_WC; ++c) {
        const float sa = __shfl_sync(0xffffffffu, mine, 2 * c);
        const float sb = __shfl_sync(0xffffffffu, mine, 2 * (SCAN_WC + c));
        const float v = vs[tt * SCAN_COLS + warp * SCAN_WC + c];
        // after the decay the state reads g a; the write u = beta (v - g a); the read-out sees it
        const float u = beta * (v - decay * sa);
        if (lane == 0 && j0 + c < P)
          a.o[(size_t)(t0 + tt) * width + (size_t)head * P + j0 + c] = fmaf(kq, u, decay * sb);
#pragma unroll
        for (int e = 0; e < NPL; ++e) S[e][c] = fmaf(kv[e], u, decay * S[e][c]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < NPL; ++e) {
    const int n = lane + 32 * e;
#pragma unroll
    for (int c = 0; c < SCAN_WC; ++c)
      if (n < D && j0 + c < P) st[(size_t)n * P + j0 + c] = S[e][c];
  }
}

// --------------------------------------------------------------------- gated norm
// A row of `width` float32 values in `groups` equal parts, each divided by its own root mean
// square; times weight[i % weight_len]; a gate silu(z) on the values before the norm
// (gate_first) or on the result.  One warp per (token, group).
template <typename AT>
__global__ void __launch_bounds__(128) gated_norm_kernel(const float* __restrict__ y, const AT* __restrict__ z,
                                                         long long ldz, const float* __restrict__ weight,
                                                         int weight_len, AT* __restrict__ out, int T, int width,
                                                         int groups, float eps, int gate_first) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)T * groups) return;
  const int t = (int)(item / groups), grp = (int)(item % groups);
  const int size = width / groups, base = grp * size;
  const float* row = y + (size_t)t * width + base;
  const AT* gate = z + (size_t)t * ldz + base;
  float ss = 0.f;
  for (int i = lane; i < size; i += 32) {
    float v = row[i];
    if (gate_first) v *= silu_f(to_float(gate[i]));
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)size + eps);
  AT* dst = out + (size_t)t * width + base;
  for (int i = lane; i < size; i += 32) {
    const float gv = silu_f(to_float(gate[i]));
    float v = row[i];
    if (gate_first) v *= gv;
    v = v * inv * weight[(base + i) % weight_len];
    if (!gate_first) v *= gv;
    dst[i] = from_float<AT>(v);
  }
}

template <typename AT, int NPL>
static int launch_ssd(const SsdArgs& a, int S, cudaStream_t stream) {
  const size_t smem = (size_t)(SCAN_CHUNK * (2 * a.N + SCAN_COLS) + 2 * SCAN_CHUNK) * sizeof(float);
  if (smem > 48 * 1024) return FT_ERR_SHAPE;
  const dim3 grid((a.P + SCAN_COLS - 1) / SCAN_COLS, a.heads, S);
  cudaError_t e = launch_pdl(ssd_scan_kernel<AT, NPL>, grid, dim3(SCAN_WARPS * 32), smem, stream, a);
  return e == cudaSuccess ? FT_OK : (int)e;
}

template <typename AT, int NPL>
static int launch_delta(const DeltaArgs& a, int S, cudaStream_t stream) {
  const size_t smem = (size_t)(SCAN_CHUNK * (2 * a.D + SCAN_COLS) + 3 * SCAN_CHUNK) * sizeof(float);
  if (smem > 48 * 1024) return FT_ERR_SHAPE;
  const dim3 grid((a.P + SCAN_COLS - 1) / SCAN_COLS, a.heads, S);
  cudaError_t e = launch_pdl(delta_scan_kernel<AT, NPL>, grid, dim3(SCAN_WARPS * 32), smem, stream, a);
  return e == cudaSuccess ? FT_OK : (int)e;
}

}  // namespace ft

using namespace ft;

extern "C" {

// Both kernels of the short convolution: outputs first, then the slots' new contents.
int ft_conv_silu(const void* x, long long ldx, void* out, long long ldo, const float* w, const float* bias,
                 float* state, long long slot_stride, const int* token_seg, const int* seg_slot,
                 const int* seg_q_start, int C, int taps, int T, int S, int dtype, cudaStream_t stream) {
  if (T <= 0 || S <= 0) return FT_OK;
  if (C <= 0 || taps < 1) return FT_ERR_SHAPE;
  ConvArgs a{x, out, w, bias, state, token_seg, seg_slot, seg_q_start, ldx, ldo, slot_stride, C, taps};
  const int cb = (C + 127) / 128;
  FT_DISPATCH(dtype, AT, launch_pdl(conv_silu_kernel<AT>, dim3(T, cb), dim3(128), 0, stream, a));
  FT_LAUNCH_CHECK();
  if (taps > 1) {
    FT_DISPATCH(dtype, AT, launch_pdl(conv_state_kernel<AT>, dim3(S, cb), dim3(128), 0, stream, a));
    FT_LAUNCH_CHECK();
  }
  return FT_OK;
}

int ft_ssd_scan(const void* xbc, long long ld, const void* dt, long long ld_dt, const float* dt_bias,
                const float* A_log, const float* D, float* state, long long slot_stride, float* y,
                const int* seg_slot, const int* seg_q_start, int heads, int P, int N, int G, int S,
                int dtype, cudaStream_t stream) {
  if (S <= 0) return FT_OK;
  if (heads <= 0 || P <= 0 || N <= 0 || N > 256 || G <= 0 || heads % G) return FT_ERR_SHAPE;
  SsdArgs a{xbc, dt, dt_bias, A_log, D, state, y, seg_slot, seg_q_start, ld, ld_dt, slot_stride, heads, P, N, G};
  int rc = FT_OK;
  FT_DISPATCH(dtype, AT, {
    if (N <= 32) rc = launch_ssd<AT, 1>(a, S, stream);
    else if (N <= 64) rc = launch_ssd<AT, 2>(a, S, stream);
    else if (N <= 128) rc = launch_ssd<AT, 4>(a, S, stream);
    else rc = launch_ssd<AT, 8>(a, S, stream);
  });
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_delta_scan(const void* qkv, long long ld, const void* beta, const void* decay, long long ld_gate,
                  const float* dt_bias, const float* A_log, float* state, long long slot_stride, float* o,
                  const int* seg_slot, const int* seg_q_start, int heads, int P, int D, int G, float unit_eps,
                  float q_scale, int S, int dtype, cudaStream_t stream) {
  if (S <= 0) return FT_OK;
  if (heads <= 0 || P <= 0 || D <= 0 || D > 256 || G <= 0 || heads % G) return FT_ERR_SHAPE;
  DeltaArgs a{qkv, beta, decay, dt_bias, A_log, state, o, seg_slot, seg_q_start, ld, ld_gate, slot_stride,
              heads, P, D, G, unit_eps, q_scale};
  int rc = FT_OK;
  FT_DISPATCH(dtype, AT, {
    if (D <= 32) rc = launch_delta<AT, 1>(a, S, stream);
    else if (D <= 64) rc = launch_delta<AT, 2>(a, S, stream);
    else if (D <= 128) rc = launch_delta<AT, 4>(a, S, stream);
    else rc = launch_delta<AT, 8>(a, S, stream);
  });
  if (rc != FT_OK) return rc;
  FT_LAUNCH_CHECK();
  return FT_OK;
}

int ft_gated_norm(const float* y, const void* z, long long ldz, const float* weight, int weight_len, void* out,
                  int T, int width, int groups, float eps, int gate_first, int dtype, cudaStream_t stream) {
  if (T <= 0) return FT_OK;
  if (width <= 0 || groups <= 0 || width % groups || weight_len <= 0) return FT_ERR_SHAPE;
  const long long items = (long long)T * groups;
  const unsigned blocks = (unsigned)((items + 3) / 4);
  FT_DISPATCH(dtype, AT, launch_pdl(gated_norm_kernel<AT>, dim3(blocks), dim3(128), 0, stream, y, (const AT*)z, ldz,
                                    weight, weight_len, (AT*)out, T, width, groups, eps, gate_first));
  FT_LAUNCH_CHECK();
  return FT_OK;
}

}  // extern "C"

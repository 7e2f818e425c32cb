// Linear attention with a constant decay per head, as a recurrence over a state of fixed size
// per request, and the gated RMSNorm that follows it.
//
// Per sequence and head, with q_t, k_t of size dim and v_t of size vdim (read from a stacked
// projection row and passed through an activation on the way in):
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        S is [dim, vdim], 32-bit, kept in the request's state slot
//   o_t = S_t^T q_t                            o_t[e] = sum_d S_t[d, e] q_t[d]
//
// One kernel serves a whole prompt, a portion of one and a single decoded token: a sequence's
// tokens of the step are walked in order from the state the step before left, and the new state
// is written back. Every state element follows the same sequence of operations whatever the cut
// (s = fma(k, v, decay * s); the sum over d is taken in a fixed order), so the result does not
// depend on how the tokens were cut into steps or on what else is in the batch, bit for bit.
// State, decay, products and sums are 32-bit; only q, k, v arrive in the run's type T.
//
// Grid (ceil(vdim / 32), heads, sequences), 256 threads: warp r owns rows [r * DPT, (r + 1) * DPT)
// of S, lane j column blockIdx.x * 32 + j, so a thread keeps DPT state elements in registers and
// never synchronises inside a token. Tokens are taken CHUNK at a time: q, k, v of the chunk go to
// shared memory (k and q are read as broadcasts), each warp leaves its partial sums of o per token,
// and the eight partial sums are added in warp order at the end of the chunk.
#include <math.h>

#include "common.cuh"

namespace {
constexpr int RANGES = 8;     // warps: ranges of state rows
constexpr int COLS = 32;      // value columns per block (one per lane)

template <int ACT> __device__ __forceinline__ float activate(float z) {
  return ACT == 1 ? z / (1.0f + expf(-z)) : z;      // 1: silu, 0: none
}

template <typename T, int DPT, int ACT>
__global__ void __launch_bounds__(RANGES * COLS)
decay_scan_kernel(const T* __restrict__ proj, long row_stride, int q_off, int k_off, int v_off,
                  float* __restrict__ out, float* __restrict__ state, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, const float* __restrict__ decay, int heads, int dim, int vdim) {
  constexpr int DPAD = RANGES * DPT;
  constexpr int CHUNK = DPT >= 32 ? 8 : 16;     // tokens per trip through shared memory (under 48 KB in all)
  __shared__ __align__(16) float q_s[CHUNK][DPAD];
  __shared__ __align__(16) float k_s[CHUNK][DPAD];
  __shared__ float v_s[CHUNK][COLS];
  __shared__ float part_s[CHUNK][RANGES][COLS];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y, e0 = blockIdx.x * COLS;
  const int r = threadIdx.x >> 5, j = threadIdx.x & 31, e = e0 + j;
  const int first = cu_q[seq], count = cu_q[seq + 1] - first;
  const float lam = decay[head];
  float* mine = state + ((size_t)state_slots[seq] * heads + head) * dim * vdim;
  float s[DPT];
#pragma unroll
  for (int x = 0; x < DPT; ++x) {
    const int d = r * DPT + x;
    s[x] = (d < dim && e < vdim) ? mine[(size_t)d * vdim + e] : 0.f;
  }
  for (int t0 = 0; t0 < count; t0 += CHUNK) {
    const int n = min(CHUNK, count - t0);
    __syncthreads();                         // the partial sums of the chunk before have been read
    for (int i = threadIdx.x; i < n * DPAD; i += blockDim.x) {
      const int t = i / DPAD, d = i - t * DPAD;
      const T* row = proj + (size_t)(first + t0 + t) * row_stride;
      q_s[t][d] = d < dim ? activate<ACT>(Elem<T>::load(row + q_off + head * dim + d)) : 0.f;
      k_s[t][d] = d < dim ? activate<ACT>(Elem<T>::load(row + k_off + head * dim + d)) : 0.f;
    }
    for (int i = threadIdx.x; i < n * COLS; i += blockDim.x) {
      const int t = i / COLS, c = i - t * COLS;
      const T* row = proj + (size_t)(first + t0 + t) * row_stride;
      v_s[t][c] = e0 + c < vdim ? activate<ACT>(Elem<T>::load(row + v_off + head * vdim + e0 + c)) : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float v = v_s[t][j];
      const float* kr = &k_s[t][r * DPT];
      const float* qr = &q_s[t][r * DPT];
      float partial = 0.f;
#pragma unroll
      for (int x = 0; x < DPT; ++x) {
        s[x] = fmaf(kr[x], v, lam * s[x]);
        partial = fmaf(s[x], qr[x], partial);
      }
      part_s[t][r][j] = partial;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * COLS; i += blockDim.x) {
      const int t = i / COLS, c = i - t * COLS;
      if (e0 + c >= vdim) continue;
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < RANGES; ++w) total += part_s[t][w][c];
      out[((size_t)(first + t0 + t) * heads + head) * vdim + e0 + c] = total;
    }
  }
#pragma unroll
  for (int x = 0; x < DPT; ++x) {
    const int d = r * DPT + x;
    if (d < dim && e < vdim) mine[(size_t)d * vdim + e] = s[x];
  }
}

template <typename T, int DPT>
int launch_scan(int act, dim3 grid, cudaStream_t stream, const void* proj, long row_stride, int q_off, int k_off, int v_off,
                float* out, float* state, const int* cu_q, const int* state_slots, const float* decay, int heads,
                int dim, int vdim) {
  if (act == 1)
    lb_launch(decay_scan_kernel<T, DPT, 1>, grid, RANGES * COLS, 0, stream, (const T*)proj, row_stride, q_off, k_off, v_off,
              out, state, cu_q, state_slots, decay, heads, dim, vdim);
  else
    lb_launch(decay_scan_kernel<T, DPT, 0>, grid, RANGES * COLS, 0, stream, (const T*)proj, row_stride, q_off, k_off, v_off,
              out, state, cu_q, state_slots, decay, heads, dim, vdim);
  return lb_last_error();
}

template <typename T>
int dispatch_scan(int act, dim3 grid, cudaStream_t stream, const void* proj, long row_stride, int q_off, int k_off,
                  int v_off, float* out, float* state, const int* cu_q, const int* state_slots, const float* decay,
                  int heads, int dim, int vdim) {
#define LB_SCAN(D) launch_scan<T, D>(act, grid, stream, proj, row_stride, q_off, k_off, v_off, out, state, cu_q, state_slots, \
                                     decay, heads, dim, vdim)
  if (dim <= RANGES * 4) return LB_SCAN(4);
  if (dim <= RANGES * 8) return LB_SCAN(8);
  if (dim <= RANGES * 16) return LB_SCAN(16);
  return LB_SCAN(32);
#undef LB_SCAN
}

// out[t, i] = T(x[t, i] * rsqrt(mean_i x[t, i]^2 + eps) * weight[i] / (1 + exp(-gate[t, i])))
// x 32-bit [tokens, n]; gate logits in the run's type inside a wider row (gate_stride elements apart).
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ x, const T* __restrict__ gate, long gate_stride,
                                     const float* __restrict__ weight, T* __restrict__ out, int n, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* xr = x + (size_t)blockIdx.x * n;
  const T* gr = gate + (size_t)blockIdx.x * gate_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
  T* o = out + (size_t)blockIdx.x * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    Elem<T>::store(o + i, xr[i] * inv * weight[i] / (1.0f + expf(-Elem<T>::load(gr + i))));
}
}  // namespace

// proj [tokens, row_stride] holds q at q_off (heads * dim), k at k_off (heads * dim), v at v_off (heads * vdim);
// out float [tokens, heads * vdim]; state float [slots, heads, dim, vdim]; decay float [heads]; act 0 none, 1 silu.
LB_EXPORT int lb_decay_scan(int dtype, const void* proj, long row_stride, int q_off, int k_off, int v_off, float* out,
                            float* state, const int* cu_q, const int* state_slots, const float* decay, int n_seqs,
                            int heads, int dim, int vdim, int act, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || heads > 65535 || n_seqs > 65535 || dim <= 0 || dim > RANGES * 32 || vdim <= 0 || act < 0 || act > 1)
    return LB_ERR_SIZE;
  const dim3 grid((vdim + COLS - 1) / COLS, heads, n_seqs);
  if (dtype == LB_F32)
    return dispatch_scan<float>(act, grid, stream, proj, row_stride, q_off, k_off, v_off, out, state, cu_q, state_slots,
                                decay, heads, dim, vdim);
  if (dtype == LB_BF16)
    return dispatch_scan<bf16>(act, grid, stream, proj, row_stride, q_off, k_off, v_off, out, state, cu_q, state_slots,
                               decay, heads, dim, vdim);
  return LB_ERR_DTYPE;
}

LB_EXPORT int lb_gated_rmsnorm(int dtype, const float* x, const void* gate, long gate_stride, const float* weight,
                               void* out, int tokens, int n, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n <= 0) return LB_ERR_SIZE;
  const int threads = n >= 1024 ? 256 : 128;
  if (dtype == LB_F32)
    lb_launch(gated_rmsnorm_kernel<float>, tokens, threads, 0, stream, x, (const float*)gate, gate_stride, weight,
              (float*)out, n, eps);
  else if (dtype == LB_BF16)
    lb_launch(gated_rmsnorm_kernel<bf16>, tokens, threads, 0, stream, x, (const bf16*)gate, gate_stride, weight,
              (bf16*)out, n, eps);
  else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

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
// Grid (ceil(vdim / 32), heads, sequences), RANGES warps: warp r owns rows [r * DPT, (r + 1) * DPT) of
// S, lane j column blockIdx.x * 32 + j, so a thread keeps DPT state elements in registers and never
// synchronises inside a token. Tokens are taken CHUNK (8) at a time through two buffers in shared
// memory: while a chunk is computed (k and q are read as 16-byte broadcasts, each warp leaves its
// partial sums of o per token), the next chunk's q, k, v are already on their way from global
// memory into registers; the warps' partial sums are added in warp order at the end of the chunk.
// RANGES and DPT depend on the head size only, never on the batch.
//
// A long portion of one sequence is a long chain for few blocks. Steps that hold one (the host
// decides from the step's longest portion) run in three launches instead: every sequence's portion
// is cut into segments of `seg_tokens`; MODE 1 scans every segment at once, a sequence's first
// segment from the slot's state and the others from zero, and leaves each segment's end state in
// `seg_state`; the combine kernel walks a sequence's segments in order, S_in(s+1) = decay^len(s)
// S_in(s) + S_end(s), leaves S_in(s) where segment s finds it and the last one in the slot; MODE 2
// adds what the incoming state contributes, o_t += decay^(t+1) S_in^T q_t for the t-th token of the
// segment. The sums are the same numbers in another order: results agree with the single pass
// within rounding, not bit for bit.
#include <math.h>

#include "common.cuh"

namespace {
constexpr int COLS = 32;      // value columns per block (one per lane)
constexpr int CHUNK = 8;      // tokens per trip through shared memory (a thread stages at most one value of v: CHUNK * 32 <= threads)

template <int ACT> __device__ __forceinline__ float activate(float z) {
  return ACT == 1 ? z / (1.0f + __expf(-z)) : z;      // 1: silu, 0: none
}

// the sequence and the segment of it that global segment `g` is; a sequence has at least one segment
__device__ __forceinline__ void find_segment(const int* __restrict__ cu_q, int n_seqs, int seg_tokens, int g, int& seq,
                                             int& segment, int& first_segment) {
  seq = 0;
  first_segment = 0;
  for (; seq < n_seqs - 1; ++seq) {
    const int len = cu_q[seq + 1] - cu_q[seq], ns = max(1, (len + seg_tokens - 1) / seg_tokens);
    if (g < first_segment + ns) break;
    first_segment += ns;
  }
  segment = g - first_segment;
}

template <typename T, int RANGES, int DPT, int ACT, int MODE = 0>
__global__ void __launch_bounds__(RANGES * COLS)
decay_scan_kernel(const T* __restrict__ proj, long row_stride, int q_off, int k_off, int v_off,
                  float* __restrict__ out, float* __restrict__ state, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, const float* __restrict__ decay, int heads, int dim, int vdim,
                  float* __restrict__ seg_state, int seg_tokens, int n_seqs) {
  static_assert(DPT % 4 == 0, "16-byte broadcasts");
  static_assert(CHUNK * COLS <= RANGES * COLS, "one value of v per staging thread");
  constexpr int DPAD = RANGES * DPT, THREADS = RANGES * COLS;
  constexpr int QK_EACH = (CHUNK * DPAD + THREADS - 1) / THREADS;     // q (and k) elements a thread stages per chunk
  extern __shared__ __align__(16) float scan_smem[];
  float (*q_s)[CHUNK][DPAD] = reinterpret_cast<float (*)[CHUNK][DPAD]>(scan_smem);                       // [2][CHUNK][DPAD]
  float (*k_s)[CHUNK][DPAD] = reinterpret_cast<float (*)[CHUNK][DPAD]>(scan_smem + 2 * CHUNK * DPAD);    // [2][CHUNK][DPAD]
  float (*v_s)[CHUNK][COLS] = reinterpret_cast<float (*)[CHUNK][COLS]>(scan_smem + 4 * CHUNK * DPAD);    // [2][CHUNK][COLS]
  float (*part_s)[RANGES][COLS] = reinterpret_cast<float (*)[RANGES][COLS]>(scan_smem + 4 * CHUNK * DPAD + 2 * CHUNK * COLS);
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.y, e0 = blockIdx.x * COLS;
  const int r = threadIdx.x >> 5, j = threadIdx.x & 31, e = e0 + j;
  int seq = blockIdx.z, segment = 0, first_segment = 0;
  if (MODE != 0) find_segment(cu_q, n_seqs, seg_tokens, blockIdx.z, seq, segment, first_segment);
  if (MODE == 2 && segment == 0) return;          // a first segment started from the true state: nothing to add
  const int first = cu_q[seq] + (MODE != 0 ? segment * seg_tokens : 0);
  const int count = MODE != 0 ? min(seg_tokens, cu_q[seq + 1] - first) : cu_q[seq + 1] - first;
  const float lam = decay[head];
  const float log2_lam = log2f(lam);                // -inf for a decay of 0: exp2f gives 0
  // MODE 0: from and to the slot; 1: a first segment from the slot, the others from zero, the end to seg_state;
  // 2: the state that came into this segment (left by the combine kernel in the segment before's place), frozen
  float* mine = state + ((size_t)state_slots[seq] * heads + head) * dim * vdim;
  float* kept = MODE != 0 ? seg_state + ((size_t)(blockIdx.z - (MODE == 2 ? 1 : 0)) * heads + head) * dim * vdim : nullptr;
  const float* from = MODE == 2 ? kept : ((MODE == 1 && segment > 0) ? nullptr : mine);
  float s[DPT];
#pragma unroll
  for (int x = 0; x < DPT; ++x) {
    const int d = r * DPT + x;
    s[x] = (from && d < dim && e < vdim) ? from[(size_t)d * vdim + e] : 0.f;
  }
  // what this thread fetches of a chunk: QK_EACH elements of q and of k, and (the first CHUNK * 32 threads) one of v
  float q_reg[QK_EACH], k_reg[QK_EACH], v_reg = 0.f;
  auto fetch = [&](int t0, int n) {
#pragma unroll
    for (int u = 0; u < QK_EACH; ++u) {
      const int i = threadIdx.x + u * THREADS, t = i / DPAD, d = i - t * DPAD;
      q_reg[u] = k_reg[u] = 0.f;
      if (t < n && d < dim) {
        const T* row = proj + (size_t)(first + t0 + t) * row_stride + head * dim + d;
        q_reg[u] = Elem<T>::load(row + q_off);
        if (MODE != 2) k_reg[u] = Elem<T>::load(row + k_off);
      }
    }
    if (MODE != 2 && threadIdx.x < CHUNK * COLS) {
      const int t = threadIdx.x / COLS, c = threadIdx.x - t * COLS;
      v_reg = (t < n && e0 + c < vdim)
                  ? Elem<T>::load(proj + (size_t)(first + t0 + t) * row_stride + v_off + head * vdim + e0 + c) : 0.f;
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int u = 0; u < QK_EACH; ++u) {
      const int i = threadIdx.x + u * THREADS, t = i / DPAD, d = i - t * DPAD;
      if (t < CHUNK) {
        q_s[buf][t][d] = activate<ACT>(q_reg[u]);
        k_s[buf][t][d] = activate<ACT>(k_reg[u]);
      }
    }
    if (threadIdx.x < CHUNK * COLS) v_s[buf][threadIdx.x / COLS][threadIdx.x % COLS] = activate<ACT>(v_reg);
  };
  fetch(0, min(CHUNK, count));
  stage(0);
  __syncthreads();
  int buf = 0;
  for (int t0 = 0; t0 < count; t0 += CHUNK, buf ^= 1) {
    const int n = min(CHUNK, count - t0);
    const bool more = t0 + CHUNK < count;
    if (more) fetch(t0 + CHUNK, min(CHUNK, count - t0 - CHUNK));     // in flight while this chunk is computed
#pragma unroll 2
    for (int t = 0; t < n; ++t) {
      const float v = v_s[buf][t][j];
      const float4* kr = reinterpret_cast<const float4*>(&k_s[buf][t][r * DPT]);
      const float4* qr = reinterpret_cast<const float4*>(&q_s[buf][t][r * DPT]);
      float partial[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int x4 = 0; x4 < DPT / 4; ++x4) {
        const float4 k4 = kr[x4], q4 = qr[x4];
        if (MODE != 2) {
          s[4 * x4 + 0] = fmaf(k4.x, v, lam * s[4 * x4 + 0]);
          s[4 * x4 + 1] = fmaf(k4.y, v, lam * s[4 * x4 + 1]);
          s[4 * x4 + 2] = fmaf(k4.z, v, lam * s[4 * x4 + 2]);
          s[4 * x4 + 3] = fmaf(k4.w, v, lam * s[4 * x4 + 3]);
        }
        partial[0] = fmaf(s[4 * x4 + 0], q4.x, partial[0]);
        partial[1] = fmaf(s[4 * x4 + 1], q4.y, partial[1]);
        partial[2] = fmaf(s[4 * x4 + 2], q4.z, partial[2]);
        partial[3] = fmaf(s[4 * x4 + 3], q4.w, partial[3]);
      }
      part_s[t][r][j] = (partial[0] + partial[1]) + (partial[2] + partial[3]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * COLS; i += THREADS) {
      const int t = i / COLS, c = i - t * COLS;
      if (e0 + c >= vdim) continue;
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < RANGES; ++w) total += part_s[t][w][c];
      float* at = out + ((size_t)(first + t0 + t) * heads + head) * vdim + e0 + c;
      if (MODE == 2) *at += exp2f((float)(t0 + t + 1) * log2_lam) * total;
      else *at = total;
    }
    if (more) stage(buf ^ 1);
    __syncthreads();      // the partial sums have been read, the next chunk is in place
  }
  if (MODE == 2) return;
  float* to = MODE == 1 ? kept : mine;
#pragma unroll
  for (int x = 0; x < DPT; ++x) {
    const int d = r * DPT + x;
    if (d < dim && e < vdim) to[(size_t)d * vdim + e] = s[x];
  }
}

// Per sequence, head and state element: the segments' end states become the states that come INTO the
// segments (left in the place of the segment before), and the state after the last segment goes to the slot.
__global__ void scan_combine_kernel(float* __restrict__ seg_state, float* __restrict__ state, const int* __restrict__ cu_q,
                                    const int* __restrict__ state_slots, const float* __restrict__ decay, int heads,
                                    int per_head, int seg_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, per_segment = (size_t)heads * per_head;
  if (i >= per_segment) return;
  int first_segment = 0;
  for (int q = 0; q < seq; ++q) first_segment += max(1, (cu_q[q + 1] - cu_q[q] + seg_tokens - 1) / seg_tokens);
  const int len = cu_q[seq + 1] - cu_q[seq], ns = max(1, (len + seg_tokens - 1) / seg_tokens);
  const float log2_lam = log2f(decay[i / per_head]);
  float* e = seg_state + (size_t)first_segment * per_segment + i;
  float running = e[0];                              // the true state after the first segment
  for (int sg = 1; sg < ns; ++sg) {
    const float local = e[(size_t)sg * per_segment];
    e[(size_t)(sg - 1) * per_segment] = running;     // what comes into segment sg
    running = fmaf(exp2f((float)min(seg_tokens, len - sg * seg_tokens) * log2_lam), running, local);
  }
  state[(size_t)state_slots[seq] * per_segment + i] = running;
}

template <typename T, int RANGES, int DPT, int ACT, int MODE>
int launch_scan_mode(dim3 grid, cudaStream_t stream, const void* proj, long row_stride, int q_off, int k_off, int v_off,
                     float* out, float* state, const int* cu_q, const int* state_slots, const float* decay, int heads,
                     int dim, int vdim, float* seg_state, int seg_tokens, int n_seqs) {
  // q and k twice (two buffers), v twice, the warps' partial sums
  constexpr size_t smem = (size_t)(4 * CHUNK * RANGES * DPT + 2 * CHUNK * COLS + CHUNK * RANGES * COLS) * sizeof(float);
  static LbPerDeviceOnce once;
  if (smem > 48 * 1024 && once.first())
    cudaFuncSetAttribute(decay_scan_kernel<T, RANGES, DPT, ACT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  lb_launch(decay_scan_kernel<T, RANGES, DPT, ACT, MODE>, grid, RANGES * COLS, smem, stream, (const T*)proj, row_stride, q_off,
            k_off, v_off, out, state, cu_q, state_slots, decay, heads, dim, vdim, seg_state, seg_tokens, n_seqs);
  return lb_last_error();
}

template <typename T, int RANGES, int DPT, int ACT>
int launch_scan(int n_seqs, int total_segments, int seg_tokens, float* seg_state, cudaStream_t stream, const void* proj,
                long row_stride, int q_off, int k_off, int v_off, float* out, float* state, const int* cu_q,
                const int* state_slots, const float* decay, int heads, int dim, int vdim) {
  const unsigned cols = (vdim + COLS - 1) / COLS;
#define LB_MODE(M, Z) launch_scan_mode<T, RANGES, DPT, ACT, M>(dim3(cols, heads, Z), stream, proj, row_stride, q_off, k_off, \
                                                                v_off, out, state, cu_q, state_slots, decay, heads, dim, vdim, \
                                                                seg_state, seg_tokens, n_seqs)
  if (total_segments <= 0) return LB_MODE(0, n_seqs);
  int code = LB_MODE(1, total_segments);
  if (code) return code;
  const int per_head = dim * vdim;
  lb_launch(scan_combine_kernel, dim3((unsigned)(((size_t)heads * per_head + 255) / 256), n_seqs), 256, 0, stream, seg_state,
            state, cu_q, state_slots, decay, heads, per_head, seg_tokens);
  if ((code = lb_last_error())) return code;
  return LB_MODE(2, total_segments);
#undef LB_MODE
}

template <typename T>
int dispatch_scan(int act, int n_seqs, int total_segments, int seg_tokens, float* seg_state, cudaStream_t stream,
                  const void* proj, long row_stride, int q_off, int k_off, int v_off, float* out, float* state,
                  const int* cu_q, const int* state_slots, const float* decay, int heads, int dim, int vdim) {
#define LB_SCAN(R, D)                                                                                                        \
  (act == 1 ? launch_scan<T, R, D, 1>(n_seqs, total_segments, seg_tokens, seg_state, stream, proj, row_stride, q_off, k_off, \
                                      v_off, out, state, cu_q, state_slots, decay, heads, dim, vdim)                         \
            : launch_scan<T, R, D, 0>(n_seqs, total_segments, seg_tokens, seg_state, stream, proj, row_stride, q_off, k_off, \
                                      v_off, out, state, cu_q, state_slots, decay, heads, dim, vdim))
  if (dim <= 32) return LB_SCAN(8, 4);          // the split of S over warps is a function of the head size alone
  if (dim <= 64) return LB_SCAN(16, 4);
  if (dim <= 128) return LB_SCAN(16, 8);
  return LB_SCAN(8, 32);
#undef LB_SCAN
}

// out[t, i] = T(x[t, i] * rsqrt(mean_i x[t, i]^2 + eps) * weight[i] / (1 + exp(-gate[t, i])))
// x 32-bit [tokens, n]; gate logits in the run's type inside a wider row (gate_stride elements apart).
template <typename T, bool VEC>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ x, const T* __restrict__ gate, long gate_stride,
                                     const float* __restrict__ weight, T* __restrict__ out, int n, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* xr = x + (size_t)blockIdx.x * n;
  const T* gr = gate + (size_t)blockIdx.x * gate_stride;
  T* o = out + (size_t)blockIdx.x * n;
  float ss = 0.f;
  if (VEC) {        // n a multiple of 4, rows on 16-byte (bf16: 8-byte) boundaries
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
  if (VEC) {
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i), w = *reinterpret_cast<const float4*>(weight + i);
      float g[4], y[4] = {v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) g[u] = Elem<T>::load(gr + i + u);
#pragma unroll
      for (int u = 0; u < 4; ++u) Elem<T>::store(o + i + u, y[u] / (1.0f + expf(-g[u])));
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      Elem<T>::store(o + i, xr[i] * inv * weight[i] / (1.0f + expf(-Elem<T>::load(gr + i))));
  }
}
}  // namespace

// proj [tokens, row_stride] holds q at q_off (heads * dim), k at k_off (heads * dim), v at v_off (heads * vdim);
// out float [tokens, heads * vdim]; state float [slots, heads, dim, vdim]; decay float [heads]; act 0 none, 1 silu.
// total_segments > 0: the three-launch form for steps with long portions; seg_state float
// [total_segments, heads, dim, vdim], total_segments = sum over sequences of max(1, ceil(tokens / seg_tokens)).
LB_EXPORT int lb_decay_scan(int dtype, const void* proj, long row_stride, int q_off, int k_off, int v_off, float* out,
                            float* state, const int* cu_q, const int* state_slots, const float* decay, int n_seqs,
                            int heads, int dim, int vdim, int act, float* seg_state, int seg_tokens, int total_segments,
                            cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || heads > 65535 || n_seqs > 65535 || dim <= 0 || dim > 256 || vdim <= 0 || act < 0 || act > 1)
    return LB_ERR_SIZE;
  if (total_segments > 0 && (!seg_state || seg_tokens <= 0 || total_segments < n_seqs || total_segments > 65535))
    return LB_ERR_SIZE;
  if (dtype == LB_F32)
    return dispatch_scan<float>(act, n_seqs, total_segments, seg_tokens, seg_state, stream, proj, row_stride, q_off, k_off,
                                v_off, out, state, cu_q, state_slots, decay, heads, dim, vdim);
  if (dtype == LB_BF16)
    return dispatch_scan<bf16>(act, n_seqs, total_segments, seg_tokens, seg_state, stream, proj, row_stride, q_off, k_off,
                               v_off, out, state, cu_q, state_slots, decay, heads, dim, vdim);
  return LB_ERR_DTYPE;
}

LB_EXPORT int lb_gated_rmsnorm(int dtype, const float* x, const void* gate, long gate_stride, const float* weight,
                               void* out, int tokens, int n, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n <= 0) return LB_ERR_SIZE;
  const int threads = n >= 1024 ? 256 : 128;
  const bool vec = n % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)weight % 16 == 0;
  if (dtype == LB_F32) {
    if (vec) lb_launch(gated_rmsnorm_kernel<float, true>, tokens, threads, 0, stream, x, (const float*)gate, gate_stride, weight, (float*)out, n, eps);
    else lb_launch(gated_rmsnorm_kernel<float, false>, tokens, threads, 0, stream, x, (const float*)gate, gate_stride, weight, (float*)out, n, eps);
  } else if (dtype == LB_BF16) {
    if (vec) lb_launch(gated_rmsnorm_kernel<bf16, true>, tokens, threads, 0, stream, x, (const bf16*)gate, gate_stride, weight, (bf16*)out, n, eps);
    else lb_launch(gated_rmsnorm_kernel<bf16, false>, tokens, threads, 0, stream, x, (const bf16*)gate, gate_stride, weight, (bf16*)out, n, eps);
  } else
    return LB_ERR_DTYPE;
  return lb_last_error();
}

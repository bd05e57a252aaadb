// Channel-wise gated recurrences and what stands around them: the token shift in front of a
// mixer, a short causal convolution with a bias, and the scan S_t = a_t S_(t-1) + b_t with
// gates that are functions of the current token (minGRU; the real-gated linear recurrent unit).
// Gates, decays, state and sums are 32-bit throughout; only the stored rows may be bfloat16.
//
// A request's rows are consecutive in the step (req_q_start), its state lives in its slot
// (req_slot); a prompt may be cut anywhere, a step may mix portions and single tokens.
#include <math.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float softplusf(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------- token shift --
// out[t] = x[t] + (x[t-1] - x[t]) * mu, where the row before a request's first row is its
// state (zeros for a new request).  The block of a request's first row also stores the
// request's last row as the new state: the same thread reads the old value of a channel and
// then writes the new one, and no other block reads the state.  mu == nullptr: a plain
// conversion of the rows.
template <typename O>
__global__ void __launch_bounds__(256)
token_shift_kernel(O* __restrict__ out, const float* __restrict__ x, const float* __restrict__ mu,
                   float* __restrict__ state, const int* __restrict__ row_req, const int* __restrict__ req_q_start,
                   const int* __restrict__ req_slot, int d) {
  pdl_trigger();
  const int t = blockIdx.x;
  int first = 0, last = 0, slot = 0;
  if (mu) {
    const int req = row_req[t];
    first = req_q_start[req];
    last = req_q_start[req + 1] - 1;
    slot = req_slot[req];
  }
  pdl_wait();
  const float* row = x + (size_t)t * d;
  O* dst = out + (size_t)t * d;
  if (!mu) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_float<O>(row[i]);
    return;
  }
  float* st = state + (size_t)slot * d;
  const float* before = t > first ? row - d : st;
  const float* newest = x + (size_t)last * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = row[i], p = before[i];
    dst[i] = from_float<O>(v + (p - v) * mu[i]);
    if (t == first) st[i] = newest[i];
  }
}

// ------------------------------------------------------- causal convolution --
// out[t, c] = bias[c] + sum_j w[j, c] * in(t - taps + 1 + j, c); w is tap-major.  Inputs from
// before the portion come from the request's state (the last taps - 1 inputs of earlier steps,
// oldest first, at state + slot * slot_stride + c).  One block per row.  The state is brought up
// to date by conv_state_kernel afterwards (rows of one request run in different blocks here).
constexpr int MAX_TAPS = 16;

__global__ void __launch_bounds__(256)
causal_conv_kernel(float* __restrict__ out, const float* __restrict__ in, long long in_stride,
                   const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
                   long long slot_stride, const int* __restrict__ row_req, const int* __restrict__ req_q_start,
                   const int* __restrict__ req_slot, int C, int taps) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int req = row_req[t];
  const int first = req_q_start[req];
  const float* st = state + (size_t)req_slot[req] * slot_stride;
  pdl_wait();
  const int back = taps - 1;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int s = t - back + j;
      const float v = s >= first ? in[(size_t)s * in_stride + c] : st[(size_t)(s - first + back) * C + c];
      acc = fmaf(w[(size_t)j * C + c], v, acc);
    }
    out[(size_t)t * C + c] = acc;
  }
}

// The new state of every request: its last taps - 1 inputs, oldest first.  A thread owns a
// channel of a request and moves forward through the slots, so an old value is read before
// its place is written.
__global__ void __launch_bounds__(256)
conv_state_kernel(float* __restrict__ state, long long slot_stride, const float* __restrict__ in, long long in_stride,
                  const int* __restrict__ req_q_start, const int* __restrict__ req_slot, int C, int taps) {
  pdl_trigger();
  const int req = blockIdx.y;
  const int first = req_q_start[req], end = req_q_start[req + 1];
  float* st = state + (size_t)req_slot[req] * slot_stride;
  pdl_wait();
  const int back = taps - 1;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  for (int k = 0; k < back; ++k) {
    const int s = end - back + k;
    st[(size_t)k * C + c] = s >= first ? in[(size_t)s * in_stride + c] : st[(size_t)(s - first + back) * C + c];
  }
}

// -------------------------------------------------------------------- scans --
// What a recurrence is made of: gate(t, c) gives the decay a, the input b and the factor m on
// the output, out[t, c] = S_t * m.
struct Step {
  float a, b, m;
};

// The transcendentals of the gates: the library's functions where the rows are stored in 32-bit, the
// hardware's approximations (ex2, lg2, rcp: a few ulp in 32-bit) where they are stored in bfloat16 and the
// gates' cost in issue slots is what bounds the scan.
template <bool FAST>
struct GateMath {
  static __device__ __forceinline__ float exp(float z) { return FAST ? __expf(z) : expf(z); }
  static __device__ __forceinline__ float sigmoid(float z) {
    return FAST ? __fdividef(1.0f, 1.0f + __expf(-z)) : 1.0f / (1.0f + expf(-z));
  }
  static __device__ __forceinline__ float gelu(float z) {
    return FAST ? apply_activation_tc<AYK_ACT_GELU_TANH>(z, AYK_ACT_GELU_TANH) : apply_activation(z, AYK_ACT_GELU_TANH);
  }
  // sqrt(1 - exp(2 l)) for l <= 0, without cancellation where l is close to 0
  static __device__ __forceinline__ float root_one_minus_square(float l) {
    if (!FAST) return sqrtf(-expm1f(2.0f * l));
    const float t = 2.0f * l;
    // -expm1(t): the series near zero, 1 - e^t elsewhere
    const float v = t > -0.0625f ? -t * (1.0f + t * (0.5f + t * (0.16666667f + t * 0.041666668f))) : 1.0f - __expf(t);
    return sqrtf(v);
  }
};

// minGRU over projection rows [z | u | g] (biases already added).
struct MinGruGate {
  const float* proj;
  long long stride;
  int W;
  __device__ __forceinline__ float prepare(int) const { return 0.f; }
  template <bool FAST>
  __device__ __forceinline__ Step at(int t, int c, float) const {
    typedef GateMath<FAST> M;
    const float* row = proj + (size_t)t * stride;
    const float z = M::sigmoid(row[c]);
    const float u = row[W + c];
    const float cand = u >= 0.f ? u + 0.5f : M::sigmoid(u);
    const float g = row[2 * W + c];
    return {1.0f - z, z * cand, g * M::sigmoid(g)};
  }
};

// The real-gated linear recurrent unit: proj rows [y | ...] (bias added, before its GELU), u the
// convolved branch [T, W], gates [T, blocks, r | i] before their biases, lam the decay parameter.
struct RglruGate {
  const float* proj;
  long long stride;
  const float* u;
  const float* gates;
  const float* gate_bias;
  const float* lam;
  int W, block;      // channels per block
  float decay;
  // per channel, once: -decay * softplus(lam)
  __device__ __forceinline__ float prepare(int c) const { return -decay * softplusf(lam[c]); }
  template <bool FAST>
  __device__ __forceinline__ Step at(int t, int c, float rate) const {
    typedef GateMath<FAST> M;
    const int b = c / block, j = c - b * block;
    const size_t at = (size_t)b * 2 * block + j;
    const float* g = gates + (size_t)t * 2 * W;
    const float r = M::sigmoid(g[at] + gate_bias[at]);
    const float i = M::sigmoid(g[at + block] + gate_bias[at + block]);
    const float log_a = rate * r;
    // 1 - a^2 = -expm1(2 log a): no cancellation where a is close to 1
    const float in = M::root_one_minus_square(log_a) * i * u[(size_t)t * W + c];
    return {M::exp(log_a), in, M::gelu(proj[(size_t)t * stride + c])};
  }
};

// A block takes 32 neighbouring channels of one request and walks the request's rows in spans of
// WARPS x SEG rows: every warp takes SEG consecutive rows of the span, computes their gates once
// into registers (independent loads and transcendentals, nothing waits on the recurrence) and folds
// them into (A, B) with S_end = A S_begin + B; the warps' begins follow from the state at the span's
// start by walking the folds in order; every warp then replays its rows from its true begin out of
// the registers and writes the outputs.  The state is at state + slot * slot_stride + c.
constexpr int SEG = 8;

template <typename O, typename Gate, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
scan_kernel(O* __restrict__ out, float* __restrict__ state, long long slot_stride, Gate gate,
            const int* __restrict__ req_q_start, const int* __restrict__ req_slot, int W) {
  __shared__ float fold_a[WARPS][32], fold_b[WARPS][32];
  pdl_trigger();
  const int req = blockIdx.y;
  const int first = req_q_start[req], end = req_q_start[req + 1];
  float* st = state + (size_t)req_slot[req] * slot_stride;
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 32 + lane;
  const bool live = c < W;
  constexpr bool FAST = sizeof(O) == 2;
  const float per_channel = live ? gate.prepare(c) : 0.f;
  float carry = live ? st[c] : 0.f;                     // the state at the start of the span
  for (int span = first; span < end; span += WARPS * SEG) {
    const int lo = span + warp * SEG;
    Step s[SEG];
    float A = 1.f, B = 0.f;
#pragma unroll
    for (int i = 0; i < SEG; ++i) {
      if (live && lo + i < end) s[i] = gate.template at<FAST>(lo + i, c, per_channel);
      else s[i] = Step{1.f, 0.f, 0.f};
      A *= s[i].a;
      B = fmaf(s[i].a, B, s[i].b);
    }
    float S = carry;
    if (WARPS > 1) {
      fold_a[warp][lane] = A;
      fold_b[warp][lane] = B;
      __syncthreads();
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        if (w == warp) S = carry;                       // this warp's begin: the folds before it applied
        carry = fmaf(fold_a[w][lane], carry, fold_b[w][lane]);
      }
      __syncthreads();                                  // the folds are read before the next span writes them
    } else {
      carry = fmaf(A, carry, B);
    }
#pragma unroll
    for (int i = 0; i < SEG; ++i) {
      S = fmaf(s[i].a, S, s[i].b);
      if (live && lo + i < end) out[(size_t)(lo + i) * W + c] = from_float<O>(S * s[i].m);
    }
  }
  if (live && warp == 0) st[c] = carry;
}

template <typename Gate>
int launch_scan(void* out, float* state, long long slot_stride, const Gate& gate, const int* req_q_start,
                const int* req_slot, int R, int W, int max_q_len, int out_dtype, cudaStream_t stream, const char* what) {
  dim3 grid((W + 31) / 32, R);
#define AYK_SCAN(O, WARPS)                                                                                              \
  ayk_launch(scan_kernel<O, Gate, WARPS>, grid, dim3(WARPS * 32), 0, stream, (O*)out, state, slot_stride, gate, req_q_start, \
             req_slot, W)
  // a warp per 32 channels for single tokens and short portions; 32 warps (spans of 256 rows) from 128 rows on
  if (out_dtype == AYK_DTYPE_F32) {
    if (max_q_len >= 128) AYK_SCAN(float, 32); else if (max_q_len > SEG) AYK_SCAN(float, 4); else AYK_SCAN(float, 1);
  } else if (out_dtype == AYK_DTYPE_BF16) {
    if (max_q_len >= 128) AYK_SCAN(__nv_bfloat16, 32); else if (max_q_len > SEG) AYK_SCAN(__nv_bfloat16, 4); else AYK_SCAN(__nv_bfloat16, 1);
  } else {
    return ayk_fail("%s: unknown dtype %d", what, out_dtype);
  }
#undef AYK_SCAN
  return ayk_check_launch(what);
}

// x *= factor
__global__ void scale_kernel(float* __restrict__ x, long long n, float factor) {
  pdl_trigger();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] *= factor;
}

}  // namespace

// out[T, d] (out_dtype) from the float32 rows x; mu null: a conversion only (state and the step's
// tables are not read).
AYK_EXPORT int ayk_token_shift(void* out, const float* x, const float* mu, float* state, const int* row_req,
                               const int* req_q_start, const int* req_slot, int T, int d, int out_dtype,
                               cudaStream_t stream) {
  if (T == 0 || d == 0) return 0;
  if (out_dtype == AYK_DTYPE_F32)
    ayk_launch(token_shift_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)out, x, mu, state, row_req, req_q_start,
               req_slot, d);
  else if (out_dtype == AYK_DTYPE_BF16)
    ayk_launch(token_shift_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)out, x, mu, state, row_req,
               req_q_start, req_slot, d);
  else
    return ayk_fail("ayk_token_shift: unknown dtype %d", out_dtype);
  return ayk_check_launch("ayk_token_shift");
}

// out[T, C] float32 = bias + conv(in) over time, then the state (taps - 1 rows of C per slot,
// slot_stride floats apart) is brought up to date.  Two launches.
AYK_EXPORT int ayk_causal_conv(float* out, const float* in, long long in_stride, const float* w, const float* bias,
                               float* state, long long slot_stride, const int* row_req, const int* req_q_start,
                               const int* req_slot, int T, int R, int C, int taps, cudaStream_t stream) {
  if (T == 0 || C == 0) return 0;
  AYK_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "ayk_causal_conv: %d taps are not in [1, %d]", taps, MAX_TAPS);
  ayk_launch(causal_conv_kernel, dim3(T), dim3(256), 0, stream, out, in, in_stride, w, bias, (const float*)state, slot_stride,
             row_req, req_q_start, req_slot, C, taps);
  if (taps > 1)
    ayk_launch(conv_state_kernel, dim3((C + 255) / 256, R), dim3(256), 0, stream, state, slot_stride, in, in_stride,
               req_q_start, req_slot, C, taps);
  return ayk_check_launch("ayk_causal_conv");
}

AYK_EXPORT int ayk_mingru_scan(void* out, float* state, long long slot_stride, const float* proj, long long proj_stride,
                               const int* req_q_start, const int* req_slot, int R, int T, int W, int max_q_len,
                               int out_dtype, cudaStream_t stream) {
  if (T == 0 || R == 0) return 0;
  MinGruGate gate{proj, proj_stride, W};
  return launch_scan(out, state, slot_stride, gate, req_q_start, req_slot, R, W, max_q_len, out_dtype, stream, "ayk_mingru_scan");
}

AYK_EXPORT int ayk_rglru_scan(void* out, float* state, long long slot_stride, const float* proj, long long proj_stride,
                              const float* u, const float* gates, const float* gate_bias, const float* lam, float decay,
                              const int* req_q_start, const int* req_slot, int R, int T, int W, int blocks, int max_q_len,
                              int out_dtype, cudaStream_t stream) {
  if (T == 0 || R == 0) return 0;
  AYK_REQUIRE(blocks >= 1 && W % blocks == 0, "ayk_rglru_scan: %d channels are not %d equal blocks", W, blocks);
  RglruGate gate{proj, proj_stride, u, gates, gate_bias, lam, W, W / blocks, decay};
  return launch_scan(out, state, slot_stride, gate, req_q_start, req_slot, R, W, max_q_len, out_dtype, stream, "ayk_rglru_scan");
}

AYK_EXPORT int ayk_scale(float* x, long long n, float factor, cudaStream_t stream) {
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  ayk_launch(scale_kernel, dim3(blocks), dim3(256), 0, stream, x, n, factor);
  return ayk_check_launch("ayk_scale");
}

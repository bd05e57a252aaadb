// HGRN2: a gated linear recurrence per head with a state of dim x vdim numbers,
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,   o_t = S_t^T q_t,
// where the forget gate f also says what is written (1 - f takes the place of a key).
// q = silu(z_q), f = l + (1 - l) sigmoid(z_f + b) with a lower bound l per channel; z_q, z_f and v
// are columns of one projection.  Gates, state and sums are 32-bit; the state of a request lives
// in its slot and is carried from step to step.
//
// One block: one request, one head, 32 value columns.  Lane l owns column l; the four warps each
// hold a quarter of the state's rows in registers.  Per token every thread updates its rows and
// adds up q_i S_ij over them; the four partial sums meet in shared memory (two buffers in turn, one
// barrier per token).  Gates of 16 tokens at a time are computed into shared memory first.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int WARPS = 4, COLS = 32, CHUNK = 16;

template <int DP>      // state rows per thread: ceil(dim / 4) <= DP
__global__ void __launch_bounds__(WARPS * 32)
hgrn2_kernel(float* __restrict__ out, float* __restrict__ state, const float* __restrict__ proj, int proj_stride,
             const float* __restrict__ f_bias, const float* __restrict__ lower, const int* __restrict__ req_q_start,
             const int* __restrict__ req_slot, int H, int dim, int vdim) {
  extern __shared__ float smem[];
  float* fs = smem;                         // [CHUNK][dim]
  float* qs = fs + CHUNK * dim;             // [CHUNK][dim]
  float* vs = qs + CHUNK * dim;             // [CHUNK][COLS]
  float* part = vs + CHUNK * COLS;          // [2][WARPS][COLS]
  pdl_trigger();
  const int req = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int first = req_q_start[req], n = req_q_start[req + 1] - first;
  const int slot = req_slot[req];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = c0 + lane;
  const bool col_ok = col < vdim;
  const int per = (dim + WARPS - 1) / WARPS;         // rows of this warp: [warp * per, ...)
  const int i0 = warp * per;
  pdl_wait();
  float* S = state + ((size_t)slot * H + h) * dim * vdim;
  float s[DP];
#pragma unroll
  for (int i = 0; i < DP; ++i) {
    const int row = i0 + i;
    s[i] = (i < per && row < dim && col_ok) ? S[(size_t)row * vdim + col] : 0.f;
  }
  const int qcol = h * dim, fcol = H * dim + h * dim, vcol = 2 * H * dim + h * vdim;
  for (int t0 = 0; t0 < n; t0 += CHUNK) {
    const int steps = min(CHUNK, n - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < steps * dim; i += blockDim.x) {
      const int tt = i / dim, c = i - tt * dim;
      const float* row = proj + (size_t)(first + t0 + tt) * proj_stride;
      const float zq = row[qcol + c], zf = row[fcol + c] + f_bias[h * dim + c], lo = lower[h * dim + c];
      qs[tt * dim + c] = zq / (1.0f + expf(-zq));
      fs[tt * dim + c] = lo + (1.0f - lo) * (1.0f / (1.0f + expf(-zf)));
    }
    for (int i = threadIdx.x; i < steps * COLS; i += blockDim.x) {
      const int tt = i / COLS, c = i - tt * COLS;
      vs[i] = (c0 + c < vdim) ? proj[(size_t)(first + t0 + tt) * proj_stride + vcol + c0 + c] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < steps; ++tt) {
      const float v = vs[tt * COLS + lane];
      const float* f = fs + tt * dim + i0;
      const float* q = qs + tt * dim + i0;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DP; ++i) {
        if (i < per && i0 + i < dim) {
          const float fi = f[i];
          s[i] = fmaf(fi, s[i], (1.0f - fi) * v);
          o = fmaf(q[i], s[i], o);
        }
      }
      float* mine = part + ((tt & 1) * WARPS) * COLS;
      mine[warp * COLS + lane] = o;
      __syncthreads();
      if (warp == (tt & 3) && col_ok)
        out[(size_t)(first + t0 + tt) * ((size_t)H * vdim) + h * vdim + col] =
            (mine[lane] + mine[COLS + lane]) + (mine[2 * COLS + lane] + mine[3 * COLS + lane]);
    }
  }
#pragma unroll
  for (int i = 0; i < DP; ++i) {
    const int row = i0 + i;
    if (i < per && row < dim && col_ok) S[(size_t)row * vdim + col] = s[i];
  }
}

template <int DP>
int launch(float* out, float* state, const float* proj, int proj_stride, const float* f_bias, const float* lower,
           const int* req_q_start, const int* req_slot, int R, int H, int dim, int vdim, cudaStream_t stream) {
  const size_t smem = ((size_t)2 * CHUNK * dim + CHUNK * COLS + 2 * WARPS * COLS) * sizeof(float);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(hgrn2_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return ayk_fail("ayk_hgrn2: shared memory %zu: %s", smem, cudaGetErrorString(err));
    configured = smem;
  }
  dim3 grid((vdim + COLS - 1) / COLS, H, R);
  ayk_launch(hgrn2_kernel<DP>, grid, dim3(WARPS * 32), smem, stream, out, state, proj, proj_stride, f_bias, lower,
             req_q_start, req_slot, H, dim, vdim);
  return ayk_check_launch("ayk_hgrn2");
}

}  // namespace

// out[t, h, :] = S_t^T q_t for the rows of every request of the step, in order; state
// [slots, H, dim, vdim] float32 is read at the start of a request's portion and written at its
// end.  proj [T, proj_stride] float32 holds z_q (H x dim) | z_f (H x dim) | v (H x vdim).
AYK_EXPORT int ayk_hgrn2(float* out, float* state, const float* proj, int proj_stride, const float* f_bias,
                         const float* lower, const int* req_q_start, const int* req_slot, int R, int H, int dim, int vdim,
                         cudaStream_t stream) {
  if (R == 0) return 0;
  AYK_REQUIRE(dim >= 1 && dim <= 512, "ayk_hgrn2: %d channels per head, the kernel holds up to 512", dim);
  AYK_REQUIRE(H <= 65535 && R <= 65535, "ayk_hgrn2: too many heads or requests");
  const int per = (dim + WARPS - 1) / WARPS;
  if (per <= 8) return launch<8>(out, state, proj, proj_stride, f_bias, lower, req_q_start, req_slot, R, H, dim, vdim, stream);
  if (per <= 16) return launch<16>(out, state, proj, proj_stride, f_bias, lower, req_q_start, req_slot, R, H, dim, vdim, stream);
  if (per <= 32) return launch<32>(out, state, proj, proj_stride, f_bias, lower, req_q_start, req_slot, R, H, dim, vdim, stream);
  if (per <= 64) return launch<64>(out, state, proj, proj_stride, f_bias, lower, req_q_start, req_slot, R, H, dim, vdim, stream);
  return launch<128>(out, state, proj, proj_stride, f_bias, lower, req_q_start, req_slot, R, H, dim, vdim, stream);
}

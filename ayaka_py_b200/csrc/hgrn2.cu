// HGRN2: a gated linear recurrence per head with a state of dim x vdim numbers,
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,   o_t = S_t^T q_t,
// where the forget gate f also says what is written (1 - f takes the place of a key).
// q = silu(z_q), f = l + (1 - l) sigmoid(z_f + b) with a lower bound l per channel; z_q, z_f and v
// are columns of one projection.  Gates, state and sums are 32-bit; the state of a request lives
// in its slot and is carried from step to step.
//
// Two forms.  The first walks the tokens one by one (decode steps and the reference form).  The
// second takes 16 tokens at a time (prompt portions): with b_t = sum_(r<=t) log f_r inside the chunk,
//   o_t = (q_t . e^(b_t))^T S_0 + sum_(s<=t) A_ts v_s,   A_ts = sum_i q_ti k_si e^(b_ti - b_si),  k = 1 - f,
//   S_C = diag(e^(b_C)) S_0 + sum_s (k_s . e^(b_C - b_s)) v_s^T,
// every exponent <= 0, so nothing overflows however strong the decay.  What does not depend on the
// state (gates, decays, A) is computed for all chunks side by side by a first kernel; the walk
// over a request's chunks then costs two small products per chunk.
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
  extern __shared__ __align__(16) float smem[];
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

// ------------------------------------------------------------ 16 tokens at a time --
// Two kernels.  hgrn2_chunk_prepare: one block per (chunk of 16 tokens, head), all chunks side by
// side: gates, running log-decays, and per chunk the decayed queries Q' = q e^b, the write weights
// K' = k e^(b_last - b), the chunk's decay e^(b_last) and the 16 x 16 matrix A, into scratch.
// hgrn2_chunk_scan: one block per (request, head, 16 value columns) walks the request's chunks in
// order, the state in registers (8 warps x 2 halves hold 16 slices of its rows): o = Q'^T S + A v, then S = diag(e^(b_last)) S + K' v^T.
constexpr int CT = 16, SW = 8, SC = 16;   // tokens per chunk; warps of the walk over chunks; value columns of one of its blocks
static_assert(2 * SW == CT, "each half warp finishes one token of a chunk");

// floats of scratch per (chunk, head): Q' and K' [dim][CT], the decay [dim rounded up to 4], A [CT][CT]; a multiple of 4
__host__ __device__ inline size_t chunk_floats(int dim) { return (size_t)2 * CT * dim + ((dim + 3) & ~3) + CT * CT; }

// which chunk of which request is global chunk number c?  (chunks are numbered request by request)
__device__ __forceinline__ bool find_chunk(const int* req_q_start, int num_req, int c, int& req, int& t0) {
  for (int r = 0; r < num_req; ++r) {
    const int chunks = (req_q_start[r + 1] - req_q_start[r] + CT - 1) / CT;
    if (c < chunks) { req = r; t0 = c * CT; return true; }
    c -= chunks;
  }
  return false;
}

__global__ void __launch_bounds__(128)
hgrn2_chunk_prepare_kernel(float* __restrict__ scratch, const float* __restrict__ proj, int proj_stride,
                           const float* __restrict__ f_bias, const float* __restrict__ lower,
                           const int* __restrict__ req_q_start, int num_req, int H, int dim) {
  extern __shared__ __align__(16) float smem[];
  const int ldr = dim + 1;                   // tokens that a warp reads side by side fall into different banks
  float* qs = smem;                          // [CT][ldr]  q
  float* ks = qs + CT * ldr;                 // [CT][ldr]  1 - f
  float* bs = ks + CT * ldr;                 // [CT][ldr]  running log f
  pdl_trigger();
  int req, t0;
  if (!find_chunk(req_q_start, num_req, blockIdx.x, req, t0)) return;
  const int h = blockIdx.y;
  const int first = req_q_start[req], n = req_q_start[req + 1] - first;
  const int steps = min(CT, n - t0);
  float* dst = scratch + ((size_t)blockIdx.x * H + h) * chunk_floats(dim);
  float* qfT = dst;                          // [dim][CT]
  float* kwT = qfT + (size_t)CT * dim;       // [dim][CT]
  float* gs = kwT + (size_t)CT * dim;        // [dim]
  float* As = gs + ((dim + 3) & ~3);         // [CT][CT]
  const int qcol = h * dim, fcol = H * dim + h * dim;
  pdl_wait();
  for (int i = threadIdx.x; i < CT * dim; i += blockDim.x) {
    const int tt = i / dim, c = i - tt * dim;
    float q = 0.f, k = 0.f, lf = 0.f;              // tokens beyond the portion: no decay, nothing written
    if (tt < steps) {
      const float* row = proj + (size_t)(first + t0 + tt) * proj_stride;
      const float zq = row[qcol + c], zf = row[fcol + c] + f_bias[h * dim + c], lo = lower[h * dim + c];
      const float f = lo + (1.0f - lo) * (1.0f / (1.0f + expf(-zf)));
      q = zq / (1.0f + expf(-zq));
      k = 1.0f - f;
      lf = fmaxf(logf(f), -80.0f);
    }
    qs[tt * ldr + c] = q; ks[tt * ldr + c] = k; bs[tt * ldr + c] = lf;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {        // running sums of the logs, per channel
    float run = 0.f;
    float b[CT];
#pragma unroll
    for (int tt = 0; tt < CT; ++tt) { run += bs[tt * ldr + c]; b[tt] = run; bs[tt * ldr + c] = run; }
    gs[c] = expf(run);
    float qf[CT], kw[CT];
#pragma unroll
    for (int tt = 0; tt < CT; ++tt) {
      qf[tt] = qs[tt * ldr + c] * expf(b[tt]);
      kw[tt] = ks[tt * ldr + c] * expf(run - b[tt]);
    }
#pragma unroll
    for (int u = 0; u < CT / 4; ++u) {
      reinterpret_cast<float4*>(qfT + (size_t)c * CT)[u] = make_float4(qf[4 * u], qf[4 * u + 1], qf[4 * u + 2], qf[4 * u + 3]);
      reinterpret_cast<float4*>(kwT + (size_t)c * CT)[u] = make_float4(kw[4 * u], kw[4 * u + 1], kw[4 * u + 2], kw[4 * u + 3]);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < CT * CT; e += blockDim.x) {    // A_ts for s <= t
    const int t = e / CT, sidx = e - t * CT;
    float a = 0.f;
    if (sidx <= t && t < steps) {
      const float *qt = qs + t * ldr, *kk = ks + sidx * ldr, *bt = bs + t * ldr, *bb = bs + sidx * ldr;
      for (int c = 0; c < dim; ++c) a = fmaf(qt[c] * kk[c], expf(bt[c] - bb[c]), a);
    }
    As[e] = a;
  }
}

__device__ __forceinline__ void cp_async_16(void* smem_ptr, const void* gmem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem_ptr) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem_ptr, const void* gmem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(addr), "l"(gmem_ptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DP>
__global__ void __launch_bounds__(SW * 32)
hgrn2_chunk_scan_kernel(float* __restrict__ out, float* __restrict__ state, const float* __restrict__ scratch,
                        const float* __restrict__ proj, int proj_stride, const int* __restrict__ req_q_start,
                        const int* __restrict__ req_slot, int H, int dim, int vdim) {
  extern __shared__ __align__(16) float smem[];
  const size_t per_chunk = chunk_floats(dim);              // a multiple of 4 floats
  float* stage[2] = {smem, smem + per_chunk + CT * SC};    // per buffer: the chunk's scratch, then v [CT][SC]
  float* red = smem + 2 * (per_chunk + CT * SC);           // [SW][CT][SC]
  pdl_trigger();
  const int req = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * SC;
  const int first = req_q_start[req], n = req_q_start[req + 1] - first;
  const int slot = req_slot[req];
  int chunk0 = 0;                                          // global number of the request's first chunk
  for (int r = 0; r < req; ++r) chunk0 += (req_q_start[r + 1] - req_q_start[r] + CT - 1) / CT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a block has 16 value columns; a warp's two halves hold different rows of the state: 16 slices of rows
  const int colj = lane & 15, half = lane >> 4;
  const int col = c0 + colj;
  const bool col_ok = col < vdim;
  const int per = (dim + 2 * SW - 1) / (2 * SW);
  const int i0 = (warp * 2 + half) * per;
  const int vcol = 2 * H * dim + h * vdim;
  pdl_wait();
  float* S = state + ((size_t)slot * H + h) * dim * vdim;
  float s[DP];
#pragma unroll
  for (int i = 0; i < DP; ++i) {
    const int row = i0 + i;
    s[i] = (i < per && row < dim && col_ok) ? S[(size_t)row * vdim + col] : 0.f;
  }
  const int chunks = (n + CT - 1) / CT;
  auto fetch = [&](int c, float* dst) {
    const float* src = scratch + ((size_t)(chunk0 + c) * H + h) * per_chunk;
    for (int i = threadIdx.x; i < (int)(per_chunk / 4); i += blockDim.x) cp_async_16(dst + 4 * i, src + 4 * i);
    float* v = dst + per_chunk;
    const int steps = min(CT, n - c * CT);
    for (int i = threadIdx.x; i < CT * SC; i += blockDim.x) {
      const int tt = i / SC, cc = i - tt * SC;
      if (tt < steps && c0 + cc < vdim) cp_async_4(v + i, proj + (size_t)(first + c * CT + tt) * proj_stride + vcol + c0 + cc);
      else v[i] = 0.f;
    }
    cp_async_commit();
  };
  if (chunks > 0) fetch(0, stage[0]);
  for (int c = 0; c < chunks; ++c) {
    if (c + 1 < chunks) { fetch(c + 1, stage[(c + 1) & 1]); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const float* qfT = stage[c & 1];
    const float* kwT = qfT + (size_t)CT * dim;
    const float* gs = kwT + (size_t)CT * dim;
    const float* As = gs + ((dim + 3) & ~3);
    const float* vs = stage[c & 1] + per_chunk;
    const int steps = min(CT, n - c * CT);
    float acc[CT], v[CT];
#pragma unroll
    for (int tt = 0; tt < CT; ++tt) { acc[tt] = 0.f; v[tt] = vs[tt * SC + colj]; }
#pragma unroll
    for (int i = 0; i < DP; ++i) {
      if (i < per && i0 + i < dim) {
        const float4* qf4 = reinterpret_cast<const float4*>(qfT + (size_t)(i0 + i) * CT);
        const float4* kw4 = reinterpret_cast<const float4*>(kwT + (size_t)(i0 + i) * CT);
        const float old = s[i];
        float fresh = gs[i0 + i] * old, fresh2 = 0.f;      // two chains: the sums of a row do not wait for one another
#pragma unroll
        for (int u = 0; u < CT / 4; ++u) {
          const float4 a = qf4[u], w = kw4[u];
          acc[4 * u] = fmaf(a.x, old, acc[4 * u]);
          acc[4 * u + 1] = fmaf(a.y, old, acc[4 * u + 1]);
          acc[4 * u + 2] = fmaf(a.z, old, acc[4 * u + 2]);
          acc[4 * u + 3] = fmaf(a.w, old, acc[4 * u + 3]);
          fresh = fmaf(w.x, v[4 * u], fresh);
          fresh2 = fmaf(w.y, v[4 * u + 1], fresh2);
          fresh = fmaf(w.z, v[4 * u + 2], fresh);
          fresh2 = fmaf(w.w, v[4 * u + 3], fresh2);
        }
        s[i] = fresh + fresh2;
      }
    }
#pragma unroll
    for (int tt = 0; tt < CT; ++tt) {
      acc[tt] += __shfl_xor_sync(0xffffffffu, acc[tt], 16);       // the warp's two halves
      if (half == 0) red[(warp * CT + tt) * SC + colj] = acc[tt];
    }
    __syncthreads();
    // each half warp finishes one token: the warps' partial sums (in order) plus what the chunk itself wrote
    {
      const int tt = warp * 2 + half;
      if (tt < steps) {
        float o = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < SW; ++w8) o += red[(w8 * CT + tt) * SC + colj];
        for (int sidx = 0; sidx <= tt; ++sidx) o = fmaf(As[tt * CT + sidx], vs[sidx * SC + colj], o);
        if (col_ok) out[(size_t)(first + c * CT + tt) * ((size_t)H * vdim) + h * vdim + col] = o;
      }
    }
    __syncthreads();        // the buffer and red are free for the chunk after the next
  }
#pragma unroll
  for (int i = 0; i < DP; ++i) {
    const int row = i0 + i;
    if (i < per && row < dim && col_ok) S[(size_t)row * vdim + col] = s[i];
  }
}

template <int DP>
int launch_chunk(float* out, float* state, float* scratch, const float* proj, int proj_stride, const float* f_bias,
                 const float* lower, const int* req_q_start, const int* req_slot, int R, int T, int H, int dim, int vdim,
                 cudaStream_t stream) {
  const size_t smem_p = (size_t)3 * CT * (dim + 1) * sizeof(float);
  const size_t smem_s = (2 * (chunk_floats(dim) + CT * SC) + (size_t)SW * CT * SC) * sizeof(float);
  static size_t configured_p = 48 * 1024, configured_s = 48 * 1024;
  if (smem_p > configured_p) {
    cudaError_t err = cudaFuncSetAttribute(hgrn2_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_p);
    if (err != cudaSuccess) return ayk_fail("ayk_hgrn2: shared memory %zu: %s", smem_p, cudaGetErrorString(err));
    configured_p = smem_p;
  }
  if (smem_s > configured_s) {
    cudaError_t err = cudaFuncSetAttribute(hgrn2_chunk_scan_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s);
    if (err != cudaSuccess) return ayk_fail("ayk_hgrn2: shared memory %zu: %s", smem_s, cudaGetErrorString(err));
    configured_s = smem_s;
  }
  ayk_launch(hgrn2_chunk_prepare_kernel, dim3(T / CT + R, H), dim3(128), smem_p, stream, scratch, proj, proj_stride, f_bias,
             lower, req_q_start, R, H, dim);
  if (ayk_check_launch("ayk_hgrn2 (chunk prepare)") != 0) return -1;
  ayk_launch(hgrn2_chunk_scan_kernel<DP>, dim3((vdim + SC - 1) / SC, H, R), dim3(SW * 32), smem_s, stream, out, state,
             (const float*)scratch, proj, proj_stride, req_q_start, req_slot, H, dim, vdim);
  return ayk_check_launch("ayk_hgrn2 (chunk scan)");
}

}  // namespace

// out[t, h, :] = S_t^T q_t for the rows of every request of the step, in order; state
// [slots, H, dim, vdim] float32 is read at the start of a request's portion and written at its
// end.  proj [T, proj_stride] float32 holds z_q (H x dim) | z_f (H x dim) | v (H x vdim).  scratch (or
// null): room for the form that takes 16 tokens at a time (for portions of prompts) instead of the
// walk token by token; ayk_hgrn2_scratch_floats says how much.
AYK_EXPORT int ayk_hgrn2(float* out, float* state, const float* proj, int proj_stride, const float* f_bias,
                         const float* lower, const int* req_q_start, const int* req_slot, int R, int T, int H, int dim, int vdim,
                         float* scratch, cudaStream_t stream) {
  if (R == 0) return 0;
  AYK_REQUIRE(dim >= 1 && dim <= 512, "ayk_hgrn2: %d channels per head, the kernel holds up to 512", dim);
  AYK_REQUIRE(H <= 65535 && R <= 65535, "ayk_hgrn2: too many heads or requests");
  const int per = (dim + WARPS - 1) / WARPS;
  if (scratch) {
    const int per8 = (dim + 2 * SW - 1) / (2 * SW);      // rows of the state per thread: 16 slices
#define AYK_HC(DP) return launch_chunk<DP>(out, state, scratch, proj, proj_stride, f_bias, lower, req_q_start, req_slot, R, T, H, dim, vdim, stream)
    if (per8 <= 2) AYK_HC(2);
    if (per8 <= 4) AYK_HC(4);
    if (per8 <= 8) AYK_HC(8);
    if (per8 <= 16) AYK_HC(16);
    AYK_HC(32);
#undef AYK_HC
  }
#define AYK_HG(DP) return launch<DP>(out, state, proj, proj_stride, f_bias, lower, req_q_start, req_slot, R, H, dim, vdim, stream)
  if (per <= 8) AYK_HG(8);
  if (per <= 16) AYK_HG(16);
  if (per <= 32) AYK_HG(32);
  if (per <= 64) AYK_HG(64);
  AYK_HG(128);
#undef AYK_HG
}

// Floats of scratch that the chunked form needs for a step of T rows and R requests.
AYK_EXPORT long long ayk_hgrn2_scratch_floats(int T, int R, int H, int dim) {
  return (long long)(T / CT + R) * H * (long long)chunk_floats(dim);
}

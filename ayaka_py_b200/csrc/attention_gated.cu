// Attention whose weights are a gate per key instead of a softmax over the keys, over the paged
// cache, with separate head sizes for keys and values.
//
// For the query at absolute position p of a request and the cached positions j <= p of that
// request: s_j = (q . k_j) * scale, capped as cap * tanh(s_j / cap) when cap > 0, and
// o = sum_j sigmoid(s_j + bias[head]) v_j.  Nothing is normalized over j, so partial sums over
// parts of the context simply add.  Scores, weights and sums are 32-bit.
//
// ayk_qk_norm_rotary prepares a step's rows from the float32 projection [q | k | v]: the whole
// query row and the whole key row are RMS-normed (one weight per element), the first rot_dims
// dimensions of every head are rotated by the position (dimension i with i + rot_dims/2), the
// queries go to a dense matrix, keys and values into their pages.
#include <math.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

// ----------------------------------------------------------------- prepare --
constexpr int MAX_ROT_HALF = 128;

template <typename C>
__global__ void __launch_bounds__(512)
qk_prepare_kernel(C* __restrict__ qout, C* __restrict__ kpages, C* __restrict__ vpages, const float* __restrict__ proj,
                  long long stride, const float* __restrict__ qw, const float* __restrict__ kw,
                  const float* __restrict__ freq, int rot_dims, const int* __restrict__ row_req,
                  const int* __restrict__ positions, const int* __restrict__ table, int table_stride, int page_size,
                  int H, int G, int D, int Dv, float eps, int writes) {
  __shared__ float red[32];                 // the warps' sums: queries in [0, 16), keys in [16, 32)
  __shared__ float cs[MAX_ROT_HALF], sn[MAX_ROT_HALF];
  pdl_trigger();
  const int t = blockIdx.x;
  const int p = positions[t];
  const int page = table[(size_t)row_req[t] * table_stride + p / page_size];
  pdl_wait();
  const float* q = proj + (size_t)t * stride;
  const float* k = q + (size_t)H * D;
  const float* v = k + (size_t)G * D;
  const int nq = H * D, nk = G * D, nv = G * Dv;
  const int half = rot_dims >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)p * freq[i], &sn[i], &cs[i]);
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) sq = fmaf(q[i], q[i], sq);
  for (int i = threadIdx.x; i < nk; i += blockDim.x) sk = fmaf(k[i], k[i], sk);
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red[warp] = sq; red[16 + warp] = sk; }
  __syncthreads();
  float tq = 0.f, tk = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { tq += red[w]; tk += red[16 + w]; }      // the same order in every thread
  const float inv_q = 1.0f / sqrtf(tq / (float)nq + eps);
  const float inv_k = 1.0f / sqrtf(tk / (float)nk + eps);

  C* qdst = qout + (size_t)t * nq;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) {
    const int j = i % D;
    float val = q[i] * inv_q * qw[i];
    if (j < half) {
      const float other = q[i + half] * inv_q * qw[i + half];
      val = val * cs[j] - other * sn[j];
    } else if (j < rot_dims) {
      const float other = q[i - half] * inv_q * qw[i - half];
      val = val * cs[j - half] + other * sn[j - half];
    }
    qdst[i] = from_float<C>(val);
  }
  if (!writes || page <= 0) return;
  const size_t cell = (size_t)page * page_size + (p % page_size);
  C* kdst = kpages + cell * nk;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int j = i % D;
    float val = k[i] * inv_k * kw[i];
    if (j < half) {
      const float other = k[i + half] * inv_k * kw[i + half];
      val = val * cs[j] - other * sn[j];
    } else if (j < rot_dims) {
      const float other = k[i - half] * inv_k * kw[i - half];
      val = val * cs[j - half] + other * sn[j - half];
    }
    kdst[i] = from_float<C>(val);
  }
  C* vdst = vpages + cell * nv;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) vdst[i] = from_float<C>(v[i]);
}

// ------------------------------------------------------- the general kernel --
// One block works on up to 32 consecutive rows of one request, one head and one part of the
// context: 4 warps x 8 rows.  Keys are taken 32 at a time (one per lane for the scores, one
// value column per lane for the weighted sum).  With several parts a block writes its float32
// partial sums to scratch and gated_merge_kernel adds the parts in order.
constexpr int BQ = 32;
constexpr int BKEYS = 32;
constexpr int WARPS = 4;
constexpr int RQ = BQ / WARPS;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
gated_attention_kernel(T* __restrict__ out, float* __restrict__ partial, const T* __restrict__ q,
                       const T* __restrict__ kcache, const T* __restrict__ vcache, const int* __restrict__ table,
                       int table_stride, const int* __restrict__ req_q_start, const int* __restrict__ req_pos0,
                       int num_req, int total_rows, int H, int Hkv, int D, int Dv, int page_size, float scale,
                       float cap, const float* __restrict__ head_bias, int part_keys) {
  pdl_trigger();
  pdl_wait();
  int tile = blockIdx.x, req = -1, q0 = 0, q_len = 0;
  for (int r = 0; r < num_req; ++r) {
    int len = req_q_start[r + 1] - req_q_start[r];
    int tiles = (len + BQ - 1) / BQ;
    if (tile < tiles) { req = r; q0 = tile * BQ; q_len = len; break; }
    tile -= tiles;
  }
  if (req < 0) return;
  const int h = blockIdx.y, kvh = h / (H / Hkv);
  const int rows = min(BQ, q_len - q0);
  const int row0 = req_q_start[req] + q0;
  const int pos0 = req_pos0[req] + q0;
  const int last_pos = pos0 + rows - 1;
  const int part = blockIdx.z;
  const int k_first = part_keys > 0 ? part * part_keys : 0;
  const int k_last = part_keys > 0 ? min(last_pos, k_first + part_keys - 1) : last_pos;
  if (k_first > last_pos) return;                 // the merge does not read parts beyond the context
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ldk = D + 1;
  const int ldq = (D + 3) & ~3;

  extern __shared__ float smem[];
  float* Qs = smem;                    // [BQ][ldq]
  float* Ks = Qs + BQ * ldq;           // [BKEYS][D + 1]
  float* Vs = Ks + BKEYS * ldk;        // [BKEYS][Dv]
  float* Ps = Vs + BKEYS * Dv;         // [BQ][BKEYS]

  for (int i = threadIdx.x; i < BQ * D; i += blockDim.x) {
    int r = i / D, d = i - r * D;
    Qs[r * ldq + d] = r < rows ? to_float<T>(q[(size_t)(row0 + r) * ((size_t)H * D) + h * D + d]) : 0.f;
  }
  const int NC = (Dv + 31) / 32;
  float acc[RQ][MAX_D / 32];
#pragma unroll
  for (int r = 0; r < RQ; ++r)
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) acc[r][c] = 0.f;
  const float bias = head_bias ? head_bias[h] : 0.f;
  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  const int* my_table = table + (size_t)req * table_stride;

  for (int k0 = k_first; k0 <= k_last; k0 += BKEYS) {
    __syncthreads();
    for (int i = threadIdx.x; i < BKEYS * D; i += blockDim.x) {
      int j = i / D, d = i - j * D;
      int kp = k0 + j;
      float kv = 0.f;
      if (kp <= k_last) {
        int page = my_table[kp / page_size];
        if (page > 0) kv = to_float<T>(kcache[(((size_t)page * page_size + (kp % page_size)) * Hkv + kvh) * D + d]);
      }
      Ks[j * ldk + d] = kv;
    }
    for (int i = threadIdx.x; i < BKEYS * Dv; i += blockDim.x) {
      int j = i / Dv, d = i - j * Dv;
      int kp = k0 + j;
      float vv = 0.f;
      if (kp <= k_last) {
        int page = my_table[kp / page_size];
        if (page > 0) vv = to_float<T>(vcache[(((size_t)page * page_size + (kp % page_size)) * Hkv + kvh) * Dv + d]);
      }
      Vs[j * Dv + d] = vv;
    }
    __syncthreads();

    const int kp = k0 + lane;
    const bool page_ok = kp <= k_last && my_table[kp / page_size] > 0;
#pragma unroll
    for (int r = 0; r < RQ; ++r) {
      const int row = warp * RQ + r;
      if (row >= rows) break;
      const int qpos = pos0 + row;
      const float* qr = Qs + row * ldq;
      const float* kr = Ks + lane * ldk;
      float s = 0.f;
      int d = 0;
      for (; d + 4 <= D; d += 4) {
        float4 qv = *reinterpret_cast<const float4*>(qr + d);
        s = fmaf(qv.x, kr[d], s);
        s = fmaf(qv.y, kr[d + 1], s);
        s = fmaf(qv.z, kr[d + 2], s);
        s = fmaf(qv.w, kr[d + 3], s);
      }
      for (; d < D; ++d) s = fmaf(qr[d], kr[d], s);
      s *= scale;
      if (cap > 0.f) s = cap * tanhf(s * inv_cap);
      Ps[row * BKEYS + lane] = (page_ok && kp <= qpos) ? sigmoidf(s + bias) : 0.f;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < RQ; ++r) {
      const int row = warp * RQ + r;
      if (row >= rows) break;
      const float* pr = Ps + row * BKEYS;
      for (int j = 0; j < BKEYS; ++j) {
        float p = pr[j];
        const float* vr = Vs + j * Dv;
#pragma unroll
        for (int c = 0; c < MAX_D / 32; ++c) {
          int d = lane + 32 * c;
          if (c < NC && d < Dv) acc[r][c] = fmaf(p, vr[d], acc[r][c]);
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RQ; ++r) {
    const int row = warp * RQ + r;
    if (row >= rows) break;
    const size_t at = (size_t)(row0 + row) * ((size_t)H * Dv) + h * Dv;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) {
      int d = lane + 32 * c;
      if (c < NC && d < Dv) {
        if (part_keys > 0) partial[(size_t)part * total_rows * H * Dv + at + d] = acc[r][c];
        else out[at + d] = from_float<T>(acc[r][c]);
      }
    }
  }
}

// ------------------------------------------------- the tensor-core kernel --
// bfloat16, head sizes in multiples of 16 up to 128.  The rows of a tile are (token, query head of
// one key/value head) pairs, token-major: a block of four warps holds 64 of them (16 per warp), so the
// query heads that share a key/value head also share its loads, in prompts and in single-token steps
// alike.  Keys and values come 64 at a time through two buffers of shared memory, the next tile copied
// asynchronously under the products of this one.  S = Q K^T with mma.sync m16n8k16 (float32
// sums); the weights are computed in 32-bit in the registers of S's fragments and enter the second
// product rounded to bfloat16 (as the cached values are); O stays in float32 registers.
constexpr int TC_ROWS = 64, TC_KEYS = 64;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// weight of a key: sigmoid(cap * tanh(s * scale / cap) + bias), tanh(x) = 1 - 2 / (exp(2x) + 1)
__device__ __forceinline__ float gate_weight(float s, float scale, float cap, float two_over_cap, float bias) {
  s *= scale;
  if (cap > 0.f) s = cap * (1.0f - __fdividef(2.0f, __expf(s * two_over_cap) + 1.0f));
  return __fdividef(1.0f, 1.0f + __expf(-(s + bias)));
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;                    // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int D, int DV>
__global__ void __launch_bounds__(128, 3)
gated_attention_mma_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                           const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                           const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ table, int table_stride,
                           const int* __restrict__ req_q_start, const int* __restrict__ req_pos0, int num_req,
                           int total_rows, int H, int Hkv, int page_shift, float scale, float cap,
                           const float* __restrict__ head_bias, int part_keys, int tq) {
  constexpr int LDK = D + 8, LDV = DV + 8;
  constexpr int TILE = TC_KEYS * (LDK + LDV);          // elements of one buffer: keys, then values
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* tiles = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // two buffers; the queries pass through the second first
  pdl_trigger();
  pdl_wait();
  const int hpg = H / Hkv;
  int tile = blockIdx.x, req = -1, q0 = 0, q_len = 0;
  for (int r = 0; r < num_req; ++r) {
    int len = req_q_start[r + 1] - req_q_start[r];
    int n = (len + tq - 1) / tq;
    if (tile < n) { req = r; q0 = tile * tq; q_len = len; break; }
    tile -= n;
  }
  if (req < 0) return;
  const int g = blockIdx.y;
  const int tokens = min(tq, q_len - q0);
  const int rows = tokens * hpg;                    // live rows of the tile, <= 64
  const int row0 = req_q_start[req] + q0;
  const int pos0 = req_pos0[req] + q0;
  const int last_pos = pos0 + tokens - 1;
  const int part = blockIdx.z;
  const int k_first = part_keys > 0 ? part * part_keys : 0;
  const int k_last = part_keys > 0 ? min(last_pos, k_first + part_keys - 1) : last_pos;
  if (k_first > last_pos) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int* my_table = table + (size_t)req * table_stride;
  const int page_mask = (1 << page_shift) - 1;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  // A tile of 64 keys and their values, copied asynchronously in 16-byte pieces; pieces of keys beyond the
  // part, or on the padding page, are filled with zeros.
  auto fetch = [&](int k0, int buf) {
    __nv_bfloat16* Kd = tiles + buf * TILE;
    __nv_bfloat16* Vd = Kd + TC_KEYS * LDK;
    for (int i = tid; i < TC_KEYS * (D / 8); i += 128) {
      const int j = i / (D / 8), piece = i - j * (D / 8);
      const int kp = k0 + j;
      const int page = kp <= k_last ? my_table[kp >> page_shift] : 0;
      const size_t cell = (((size_t)max(page, 0) << page_shift) + (kp & page_mask)) * Hkv + g;
      cp_async_16(Kd + j * LDK + piece * 8, kcache + cell * D + piece * 8, page > 0);
    }
    for (int i = tid; i < TC_KEYS * (DV / 8); i += 128) {
      const int j = i / (DV / 8), piece = i - j * (DV / 8);
      const int kp = k0 + j;
      const int page = kp <= k_last ? my_table[kp >> page_shift] : 0;
      const size_t cell = (((size_t)max(page, 0) << page_shift) + (kp & page_mask)) * Hkv + g;
      cp_async_16(Vd + j * LDV + piece * 8, vcache + cell * DV + piece * 8, page > 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(k_first, 0);

  // queries -> shared memory (the second buffer) -> A fragments of this warp's 16 rows
  __nv_bfloat16* Qs = tiles + TILE;
  for (int i = tid; i < TC_ROWS * (D / 8); i += 128) {
    const int m = i / (D / 8), piece = i - m * (D / 8);
    uint4 v = zero4;
    if (m < rows) {
      const int tok = m / hpg, head = g * hpg + (m - tok * hpg);
      v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + tok) * H + head) * D + piece * 8);
    }
    *reinterpret_cast<uint4*>(Qs + m * LDK + piece * 8) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const __nv_bfloat16* base = Qs + (warp * 16 + gid) * LDK + ks * 16 + tig * 2;
    qf[ks][0] = *reinterpret_cast<const uint32_t*>(base);
    qf[ks][1] = *reinterpret_cast<const uint32_t*>(base + 8 * LDK);
    qf[ks][2] = *reinterpret_cast<const uint32_t*>(base + 8);
    qf[ks][3] = *reinterpret_cast<const uint32_t*>(base + 8 * LDK + 8);
  }
  __syncthreads();                                     // the queries are in registers: the second buffer is free
  // this thread's two rows: their positions and their heads' biases
  int qpos[2];
  float bias[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = warp * 16 + gid + half * 8;
    const int tok = m / hpg;
    qpos[half] = m < rows ? pos0 + tok : -1;                       // a dead row sees nothing
    bias[half] = (head_bias && m < rows) ? head_bias[g * hpg + (m - tok * hpg)] : 0.f;
  }
  float o[DV / 8][4];
#pragma unroll
  for (int nt = 0; nt < DV / 8; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[nt][c] = 0.f;
  const float two_over_cap = cap > 0.f ? 2.0f / cap : 0.f;

  int buf = 0;
  for (int k0 = k_first; k0 <= k_last; k0 += TC_KEYS, buf ^= 1) {
    // the next tile streams into the other buffer (read last an iteration ago, behind the barrier below)
    const bool more = k0 + TC_KEYS <= k_last;
    if (more) {
      fetch(k0 + TC_KEYS, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* Ks = tiles + buf * TILE;
    const __nv_bfloat16* Vs = Ks + TC_KEYS * LDK;
    if (warp * 16 < rows) {                            // a warp without live rows only helps with the loads

    // S = Q K^T: 8 tiles of 8 keys
    float sc[TC_KEYS / 8][4];
#pragma unroll
    for (int nt = 0; nt < TC_KEYS / 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[nt][c] = 0.f;
      const __nv_bfloat16* kb = Ks + (nt * 8 + gid) * LDK + tig * 2;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        mma_bf16(sc[nt], qf[ks], *reinterpret_cast<const uint32_t*>(kb + ks * 16), *reinterpret_cast<const uint32_t*>(kb + ks * 16 + 8));
    }
    // weights, in place; fragment element c of tile nt: row gid + 8 (c / 2), key k0 + 8 nt + 2 tig + (c & 1)
    const bool edge = k0 + TC_KEYS - 1 > pos0 || k0 + TC_KEYS - 1 > k_last;
#pragma unroll
    for (int nt = 0; nt < TC_KEYS / 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = k0 + nt * 8 + tig * 2 + (c & 1);
        const float w = gate_weight(sc[nt][c], scale, cap, two_over_cap, bias[c >> 1]);
        sc[nt][c] = (edge && (key > qpos[c >> 1] || key > k_last)) || qpos[c >> 1] < 0 ? 0.f : w;
      }
    // O += P V: the 32-bit weights enter the product rounded to bfloat16, as the values they multiply are
#pragma unroll
    for (int ks = 0; ks < TC_KEYS / 16; ++ks) {
      uint32_t pf[4];
#pragma unroll
      for (int r = 0; r < 4; ++r)
        pf[r] = pack_bf16(sc[2 * ks + (r >> 1)][(r & 1) * 2], sc[2 * ks + (r >> 1)][(r & 1) * 2 + 1]);
#pragma unroll
      for (int np = 0; np < DV / 16; ++np) {
        // two value tiles (16 columns) at a time: four 8x8 matrices, transposed on the way in
        uint32_t b0, b1, b2, b3;
        const __nv_bfloat16* at = Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + np * 16 + (lane >> 4) * 8;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(at);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
        mma_bf16(o[2 * np], pf, b0, b1);
        mma_bf16(o[2 * np + 1], pf, b2, b3);
      }
    }
    }
    __syncthreads();                                   // this buffer is refilled by the fetch after the next
  }

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = warp * 16 + gid + half * 8;
    if (m >= rows) continue;
    const int tok = m / hpg, head = g * hpg + (m - tok * hpg);
    const size_t at = ((size_t)(row0 + tok) * H + head) * DV;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
      const int col = nt * 8 + tig * 2;
      if (part_keys > 0) {
        float* dst = partial + (size_t)part * total_rows * H * DV + at + col;
        dst[0] = o[nt][half * 2];
        dst[1] = o[nt][half * 2 + 1];
      } else {
        *reinterpret_cast<__nv_bfloat162*>(out + at + col) = __floats2bfloat162_rn(o[nt][half * 2], o[nt][half * 2 + 1]);
      }
    }
  }
}

// out[row] = sum over the parts that hold keys of the row's request, in order.
template <typename T>
__global__ void __launch_bounds__(256)
gated_merge_kernel(T* __restrict__ out, const float* __restrict__ partial, const int* __restrict__ row_req,
                   const int* __restrict__ positions, int total_rows, int width, int part_keys) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int used = positions[t] / part_keys + 1;
  (void)row_req;
  pdl_wait();
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float s = 0.f;
    for (int p = 0; p < used; ++p) s += partial[((size_t)p * total_rows + t) * width + i];
    out[(size_t)t * width + i] = from_float<T>(s);
  }
}

}  // namespace

AYK_EXPORT int ayk_qk_norm_rotary(void* qout, void* kpages, void* vpages, const float* proj, long long stride,
                                  const float* qw, const float* kw, const float* freq, int rot_dims, const int* row_req,
                                  const int* positions, const int* table, int table_stride, int page_size, int T, int H,
                                  int G, int D, int Dv, float eps, int writes, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  AYK_REQUIRE(rot_dims % 2 == 0 && rot_dims <= D && rot_dims / 2 <= MAX_ROT_HALF,
              "ayk_qk_norm_rotary: %d rotated dimensions do not fit a head of %d (at most %d)", rot_dims, D, 2 * MAX_ROT_HALF);
  // a row of a few thousand elements takes more warps (up to 16): with few rows in a step nothing else hides the loads
  const int threads = H * D >= 2048 ? 512 : (H * D >= 1024 ? 256 : 128);
  if (dtype == AYK_DTYPE_F32)
    ayk_launch(qk_prepare_kernel<float>, dim3(T), dim3(threads), 0, stream, (float*)qout, (float*)kpages, (float*)vpages, proj,
               stride, qw, kw, freq, rot_dims, row_req, positions, table, table_stride, page_size, H, G, D, Dv, eps, writes);
  else if (dtype == AYK_DTYPE_BF16)
    ayk_launch(qk_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (__nv_bfloat16*)qout, (__nv_bfloat16*)kpages,
               (__nv_bfloat16*)vpages, proj, stride, qw, kw, freq, rot_dims, row_req, positions, table, table_stride,
               page_size, H, G, D, Dv, eps, writes);
  else
    return ayk_fail("ayk_qk_norm_rotary: unknown dtype %d", dtype);
  return ayk_check_launch("ayk_qk_norm_rotary");
}

static int g_tensor_cores = 1;
// 0: bfloat16 steps run on the FP32 pipes too (for comparing the two kernels).
AYK_EXPORT void ayk_gated_attention_tensor_cores(int on) { g_tensor_cores = on ? 1 : 0; }

// q [T, H*D] and out [T, H*Dv] dense, of the cache's dtype.  parts > 1: the context is cut into
// parts of part_keys keys (grid z) whose partial sums go through ``partial`` [parts, T, H*Dv]
// float32 and are merged by a second launch; ``positions``: the rows' absolute positions.
AYK_EXPORT int ayk_gated_attention(void* out, float* partial, const void* q, const void* kcache, const void* vcache,
                                   const int* table, int table_stride, const int* req_q_start, const int* req_pos0,
                                   const int* row_req, const int* positions, int num_req, int total_rows, int H, int Hkv,
                                   int D, int Dv, int page_size, float scale, float cap, const float* head_bias, int parts,
                                   int part_keys, int dtype, int* launched, cudaStream_t stream) {
  if (launched) *launched = 0;
  if (num_req == 0 || total_rows == 0) return 0;
  AYK_REQUIRE(D >= 1 && D <= MAX_D && Dv >= 1 && Dv <= MAX_D, "ayk_gated_attention: head sizes %d / %d are not in [1, %d]", D, Dv, MAX_D);
  AYK_REQUIRE(Hkv >= 1 && H % Hkv == 0 && H <= 65535, "ayk_gated_attention: %d heads cannot share %d key/value heads", H, Hkv);
  AYK_REQUIRE(parts >= 1 && parts <= 65535 && (parts == 1 || (partial && part_keys > 0)), "ayk_gated_attention: bad partition");
  const int pk = parts > 1 ? part_keys : 0;
  // bfloat16 with head sizes that the tensor-core kernel holds
  const int hpg = H / Hkv;
  if (dtype == AYK_DTYPE_BF16 && g_tensor_cores && hpg <= TC_ROWS && ((D == 64 && Dv == 64) || (D == 128 && Dv == 128) ||
                                                                     (D == 64 && Dv == 128) || (D == 128 && Dv == 64) ||
                                                                     (D == 32 && Dv == 32) || (D == 16 && Dv == 16))) {
    const int tq = TC_ROWS / hpg;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    AYK_REQUIRE((1 << page_shift) == page_size, "ayk_gated_attention: pages of %d tokens are no power of two", page_size);
    dim3 grid(total_rows / tq + num_req, Hkv, parts);
#define AYK_GATED(DD, DDV)                                                                                                  \
  if (D == DD && Dv == DDV) {                                                                                               \
    const size_t smem = (size_t)2 * TC_KEYS * (DD + 8 + DDV + 8) * sizeof(__nv_bfloat16);                                   \
    static AykPerDevice granted;                                                                                            \
    if (!granted.here()) {                                                                                                  \
      cudaError_t e = cudaFuncSetAttribute(gated_attention_mma_kernel<DD, DDV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                                      \
      if (e != cudaSuccess) return ayk_fail("ayk_gated_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));     \
      granted.here() = true;                                                                                                \
    }                                                                                                                       \
    ayk_launch(gated_attention_mma_kernel<DD, DDV>, grid, dim3(128), smem, stream, (__nv_bfloat16*)out, partial,            \
               (const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, table, table_stride,    \
               req_q_start, req_pos0, num_req, total_rows, H, Hkv, page_shift, scale, cap, head_bias, pk, tq);              \
  }
    AYK_GATED(64, 64) AYK_GATED(128, 128) AYK_GATED(64, 128) AYK_GATED(128, 64) AYK_GATED(32, 32) AYK_GATED(16, 16)
#undef AYK_GATED
    if (parts > 1)
      ayk_launch(gated_merge_kernel<__nv_bfloat16>, dim3(total_rows), dim3(256), 0, stream, (__nv_bfloat16*)out,
                 (const float*)partial, row_req, positions, total_rows, H * Dv, part_keys);
    if (launched) *launched = parts > 1 ? 2 : 1;
    return ayk_check_launch("ayk_gated_attention");
  }
  const int max_tiles = total_rows / BQ + num_req;
  const size_t smem = ((size_t)BQ * ((D + 3) & ~3) + (size_t)BKEYS * (D + 1) + (size_t)BKEYS * Dv + (size_t)BQ * BKEYS) * sizeof(float);
  dim3 grid(max_tiles, H, parts);
  static size_t configured[2] = {0, 0};
  cudaError_t err;
  if (dtype == AYK_DTYPE_F32) {
    if (smem > configured[0]) {
      err = cudaFuncSetAttribute(gated_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return ayk_fail("ayk_gated_attention: shared memory %zu: %s", smem, cudaGetErrorString(err));
      configured[0] = smem;
    }
    ayk_launch(gated_attention_kernel<float>, grid, dim3(WARPS * 32), smem, stream, (float*)out, partial, (const float*)q,
               (const float*)kcache, (const float*)vcache, table, table_stride, req_q_start, req_pos0, num_req, total_rows, H,
               Hkv, D, Dv, page_size, scale, cap, head_bias, pk);
    if (parts > 1)
      ayk_launch(gated_merge_kernel<float>, dim3(total_rows), dim3(256), 0, stream, (float*)out, (const float*)partial, row_req,
                 positions, total_rows, H * Dv, part_keys);
  } else if (dtype == AYK_DTYPE_BF16) {
    if (smem > configured[1]) {
      err = cudaFuncSetAttribute(gated_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return ayk_fail("ayk_gated_attention: shared memory %zu: %s", smem, cudaGetErrorString(err));
      configured[1] = smem;
    }
    ayk_launch(gated_attention_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), smem, stream, (__nv_bfloat16*)out, partial,
               (const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, table, table_stride,
               req_q_start, req_pos0, num_req, total_rows, H, Hkv, D, Dv, page_size, scale, cap, head_bias, pk);
    if (parts > 1)
      ayk_launch(gated_merge_kernel<__nv_bfloat16>, dim3(total_rows), dim3(256), 0, stream, (__nv_bfloat16*)out,
                 (const float*)partial, row_req, positions, total_rows, H * Dv, part_keys);
  } else {
    return ayk_fail("ayk_gated_attention: unknown dtype %d", dtype);
  }
  if (launched) *launched = parts > 1 ? 2 : 1;
  return ayk_check_launch("ayk_gated_attention");
}

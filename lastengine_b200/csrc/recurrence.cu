// Linear recurrences with a matrix state per head, for packed rows of several sequences, and the
// small kernels around them.  Everything here is float: the design rule of the mixers that use it is
// that whatever enters a recurrence (decays, step sizes, write strengths, unit norms, the state) is 32-bit.
//
// The recurrence (leb_gated_recurrence), per head h with state S [d, e] and, per row t, a key k_t [d],
// a query q_t [d], a value v_t [e], a write strength w_t and a decay a_t (a number per head, or one per
// key channel):
//     S <- diag(a_t) S
//     u  = w_t v_t                    plain form (state-space layers: k = B, q = C, w = dt)
//     u  = w_t (v_t - S^T k_t)        delta form (the write replaces what the key already reads)
//     S <- S + k_t u^T
//     o_t = S^T q_t (+ skip_h v_t)
// in this order: the read-out sees the row's own write.  Several heads may share one key/query head
// (head h reads key head h / (H / Gk)).
//
// The columns of S never mix, so eight lanes own one column and walk the sequence's rows of the step in
// order; k, q, a, v and w of the rows come through shared memory.  The state is kept [slot][head][column][row] so that a warp's column is
// one contiguous run.  The same kernel serves prompts, portions and decode steps: a row's result
// depends only on the state before it and the rows of its own sequence.
#include "common.cuh"

constexpr int REC_WARPS = 4;      // warps of a block

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

constexpr int REC_ROWS = 8;       // rows of the step whose operands are staged at once
constexpr int REC_COLS = 4 * REC_WARPS;   // columns of a block: a warp walks four, eight lanes each

__device__ __forceinline__ void rec_copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rec_copy16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void rec_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void rec_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float sum8(float x) {      // over the eight lanes of a column
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

// A block is REC_COLS columns of one head of one sequence.  Eight lanes hold a column: lane j the rows
// 4 (j + 8 i) .. + 3 for i < NV, so a warp walks four columns, reads k, q and the decay of a row as 16-byte
// pieces that its four column groups share, and sums over a column in three exchanges.  The rows' operands
// come in through shared memory, REC_ROWS rows at a time in two buffers: the copies of the next rows are in
// flight while these are computed, and the walk over the rows never waits on global memory.  A staged row is
// padded with zeros to 32 NV numbers, so the walk has no bounds to test.
template <int NV, bool DELTA, bool ROW_DECAY>
__global__ void __launch_bounds__(32 * REC_WARPS)
gated_recurrence_kernel(float* __restrict__ out, int ldo, const float* __restrict__ k, const float* __restrict__ q, int ldk,
                        const float* __restrict__ v, int ldv, const float* __restrict__ wr, int ldw,
                        const float* __restrict__ decay, int ldd, const float* __restrict__ skip,
                        float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                        const int* __restrict__ seq_qlen, int H, int Gk, int d, int e, int ev, int wide) {
  extern __shared__ __align__(16) float rec_sm[];
  constexpr int DP = 32 * NV;                   // a staged row of k, q or the decay
  constexpr int DA = ROW_DECAY ? DP : 1;
  constexpr int STAGE = REC_ROWS * (2 * DP + REC_COLS) + ((REC_ROWS * (DA + 1) + 3) & ~3);
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j8 = lane & 7, cb = warp * 4 + (lane >> 3);     // place in the column, column in the block
  const int c0 = blockIdx.x * REC_COLS, c = c0 + cb;
  const bool active = c < e;
  const int h = blockIdx.y, b = blockIdx.z;
  const int slot = seq_slot[b];
  const int n = seq_qlen ? seq_qlen[b] : 1;
  const int m0 = seq_qstart[b];
  const int kh = h / (H / Gk);
  float* sp = (slot >= 0 && active) ? state + (((size_t)slot * H + h) * e + c) * d : nullptr;
  float s[4 * NV];
#pragma unroll
  for (int i = 0; i < NV; i++)
#pragma unroll
    for (int x = 0; x < 4; x++) {
      const int r = 4 * (j8 + 8 * i) + x;
      s[4 * i + x] = (sp && r < d) ? sp[r] : 0.f;
    }
  const float sk = skip ? skip[h] : 0.f;
  // one buffer: k [REC_ROWS][DP] | q [REC_ROWS][DP] | v [REC_ROWS][REC_COLS] | decay [REC_ROWS][DA] | write [REC_ROWS]
  for (int idx = threadIdx.x; idx < 2 * REC_ROWS * (DP - d); idx += blockDim.x) {      // the padding, once
    const int st = idx / (REC_ROWS * (DP - d)), rest = idx - st * (REC_ROWS * (DP - d));
    const int t = rest / (DP - d), jj = d + rest - t * (DP - d);
    float* base = rec_sm + st * STAGE;
    base[t * DP + jj] = 0.f;
    base[REC_ROWS * DP + t * DP + jj] = 0.f;
    if (ROW_DECAY) base[REC_ROWS * (2 * DP + REC_COLS) + t * DP + jj] = 0.f;
  }
  auto fetch = [&](int ch) {
    float* ks = rec_sm + (ch & 1) * STAGE;
    float* qs = ks + REC_ROWS * DP;
    float* vs = qs + REC_ROWS * DP;
    float* as = vs + REC_ROWS * REC_COLS;
    float* ws = as + REC_ROWS * DA;
    const int rows = min(REC_ROWS, n - ch * REC_ROWS);
    const size_t m = (size_t)m0 + (size_t)ch * REC_ROWS;
    if (wide) {      // every run starts on 16 bytes and d is a multiple of 4
      const int per = d / 4;
      for (int idx = threadIdx.x; idx < rows * per; idx += blockDim.x) {
        const int t = idx / per, jj = (idx - t * per) * 4;
        rec_copy16(ks + t * DP + jj, k + (m + t) * ldk + kh * d + jj);
        rec_copy16(qs + t * DP + jj, q + (m + t) * ldk + kh * d + jj);
        if (ROW_DECAY) rec_copy16(as + t * DP + jj, decay + (m + t) * ldd + h * d + jj);
      }
    } else {
      for (int idx = threadIdx.x; idx < rows * d; idx += blockDim.x) {
        const int t = idx / d, jj = idx - t * d;
        rec_copy4(ks + t * DP + jj, k + (m + t) * ldk + kh * d + jj);
        rec_copy4(qs + t * DP + jj, q + (m + t) * ldk + kh * d + jj);
        if (ROW_DECAY) rec_copy4(as + t * DP + jj, decay + (m + t) * ldd + h * d + jj);
      }
    }
    for (int idx = threadIdx.x; idx < rows * (REC_COLS + 2); idx += blockDim.x) {
      const int t = idx / (REC_COLS + 2), jj = idx - t * (REC_COLS + 2);
      if (jj < REC_COLS) {
        if (c0 + jj < ev) rec_copy4(vs + t * REC_COLS + jj, v + (m + t) * ldv + h * ev + c0 + jj);
        else if (c0 + jj < e) vs[t * REC_COLS + jj] = 1.0f;      // columns past the values' width hold a constant one
      } else if (jj == REC_COLS) {
        rec_copy4(ws + t, wr + (m + t) * ldw + h);
      } else if (!ROW_DECAY) {
        rec_copy4(as + t, decay + (m + t) * ldd + h);
      }
    }
    rec_commit();
  };
  const int n_chunks = (n + REC_ROWS - 1) / REC_ROWS;
  if (n_chunks > 0) fetch(0);
  for (int ch = 0; ch < n_chunks; ch++) {
    if (ch + 1 < n_chunks) {
      fetch(ch + 1);
      rec_wait<1>();
    } else {
      rec_wait<0>();
    }
    __syncthreads();
    const float* ks = rec_sm + (ch & 1) * STAGE;
    const float* qs = ks + REC_ROWS * DP;
    const float* vs = qs + REC_ROWS * DP;
    const float* as = vs + REC_ROWS * REC_COLS;
    const float* ws = as + REC_ROWS * DA;
    const int rows = min(REC_ROWS, n - ch * REC_ROWS);
    {
      // Every lane walks (a column group beyond e computes on whatever its place of the buffer holds and stores
      // nothing): the exchanges below name the whole warp.  The read-outs' sums over the lanes wait until the
      // buffer's rows are done and then run side by side.
      float o_part[REC_ROWS];
#pragma unroll
      for (int t = 0; t < REC_ROWS; t++) {
        o_part[t] = 0.f;
        if (t >= rows) continue;
        const float4* k4 = reinterpret_cast<const float4*>(ks + t * DP);
        const float4* q4 = reinterpret_cast<const float4*>(qs + t * DP);
        const float4* a4 = reinterpret_cast<const float4*>(as + t * DP);
        const float vc = vs[t * REC_COLS + cb], wc = ws[t];
        const float a1 = ROW_DECAY ? 0.f : as[t];
        float4 kv[NV], qv[NV];
        float dp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < NV; i++) {
          kv[i] = k4[j8 + 8 * i];
          qv[i] = q4[j8 + 8 * i];
          float4 av = make_float4(a1, a1, a1, a1);
          if (ROW_DECAY) av = a4[j8 + 8 * i];
          s[4 * i + 0] *= av.x;
          s[4 * i + 1] *= av.y;
          s[4 * i + 2] *= av.z;
          s[4 * i + 3] *= av.w;
          if (DELTA) {
            dp[0] = fmaf(s[4 * i + 0], kv[i].x, dp[0]);
            dp[1] = fmaf(s[4 * i + 1], kv[i].y, dp[1]);
            dp[2] = fmaf(s[4 * i + 2], kv[i].z, dp[2]);
            dp[3] = fmaf(s[4 * i + 3], kv[i].w, dp[3]);
          }
        }
        float u = wc * vc;
        if (DELTA) u = wc * (vc - sum8((dp[0] + dp[1]) + (dp[2] + dp[3])));
        float op[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < NV; i++) {
          s[4 * i + 0] = fmaf(kv[i].x, u, s[4 * i + 0]);
          s[4 * i + 1] = fmaf(kv[i].y, u, s[4 * i + 1]);
          s[4 * i + 2] = fmaf(kv[i].z, u, s[4 * i + 2]);
          s[4 * i + 3] = fmaf(kv[i].w, u, s[4 * i + 3]);
          op[0] = fmaf(s[4 * i + 0], qv[i].x, op[0]);
          op[1] = fmaf(s[4 * i + 1], qv[i].y, op[1]);
          op[2] = fmaf(s[4 * i + 2], qv[i].z, op[2]);
          op[3] = fmaf(s[4 * i + 3], qv[i].w, op[3]);
        }
        o_part[t] = (op[0] + op[1]) + (op[2] + op[3]);
      }
#pragma unroll
      for (int t = 0; t < REC_ROWS; t++) o_part[t] = sum8(o_part[t]);
#pragma unroll
      for (int t = 0; t < REC_ROWS; t++) {
        const size_t m = (size_t)m0 + (size_t)ch * REC_ROWS + t;
        if (t < rows && j8 == 0 && active) out[m * ldo + h * e + c] = o_part[t] + sk * vs[t * REC_COLS + cb];
      }
    }
    __syncthreads();      // the buffer is free for the rows after the next
  }
  if (sp) {
#pragma unroll
    for (int i = 0; i < NV; i++)
#pragma unroll
      for (int x = 0; x < 4; x++) {
        const int r = 4 * (j8 + 8 * i) + x;
        if (r < d) sp[r] = s[4 * i + x];
      }
  }
}

// out [M, H*e]; k, q [M, Gk*d] with the row stride ldk; v [M, H*ev]; write [M, H]; decay [M, H*d] when
// row_decay, else [M, H]; skip [H] or null; state [slots][H][e][d].  seq_qlen null: one row per sequence.
// ev < e: a head's value has ev numbers and the state's columns ev .. e-1 are written with the value one, so
// that column accumulates the keys alone (decayed and weighted like the rest) and its read-out is the
// product of that sum with the query: the normaliser of a memory whose result is divided by it.
LEB_API int leb_gated_recurrence(float* out, int ldo, const float* k, const float* q, int ldk, const float* v, int ldv,
                                 const float* write, int ldw, const float* decay, int ldd, int row_decay, int delta,
                                 const float* skip, float* state, const int* seq_slot, const int* seq_qstart,
                                 const int* seq_qlen, int B, int H, int Gk, int d, int e, int ev, cudaStream_t st) {
  if (B <= 0) return 0;
  LEB_REQUIRE(ev >= 0 && ev <= e, "leb_gated_recurrence: %d value columns for a state of %d", ev, e);
  LEB_REQUIRE(H >= 1 && Gk >= 1 && H % Gk == 0, "leb_gated_recurrence: %d heads do not divide into %d key heads", H, Gk);
  LEB_REQUIRE(d >= 1 && d <= 256 && e >= 1, "leb_gated_recurrence: a state of %d x %d (rows 1..256)", d, e);
  LEB_REQUIRE(H <= 65535 && B <= 65535, "leb_gated_recurrence: step too large");
  const dim3 grid(ceil_div(e, REC_COLS), H, B), block(32 * REC_WARPS);
  const int nv = d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 4 : 8, dp = 32 * nv;
  const size_t smem = (size_t)2 * (REC_ROWS * (2 * dp + REC_COLS) + ((REC_ROWS * ((row_decay ? dp : 1) + 1) + 3) & ~3)) * sizeof(float);
  // 16-byte copies when every run of k, q and the decay starts on 16 bytes
  const int wide = d % 4 == 0 && ldk % 4 == 0 && ((uintptr_t)k & 15) == 0 && ((uintptr_t)q & 15) == 0 &&
                   (!row_decay || (ldd % 4 == 0 && ((uintptr_t)decay & 15) == 0));
  LebPlainLaunches plain(true);
#define LEB_REC3(NV_, D_, R_)                                                                                            \
  {                                                                                                                      \
    static size_t set = 48 * 1024;                                                                                       \
    if (smem > set) {                                                                                                    \
      if (cudaFuncSetAttribute(gated_recurrence_kernel<NV_, D_, R_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return leb_fail("leb_gated_recurrence: %zu bytes of shared memory per block refused", smem);                    \
      set = smem;                                                                                                        \
    }                                                                                                                    \
    leb_launch(gated_recurrence_kernel<NV_, D_, R_>, grid, block, smem, st, out, ldo, k, q, ldk, v, ldv, write, ldw, decay, \
               ldd, skip, state, seq_slot, seq_qstart, seq_qlen, H, Gk, d, e, ev, wide);                                     \
  }
#define LEB_REC2(NV_)                                     \
  {                                                       \
    if (delta && row_decay) LEB_REC3(NV_, true, true)     \
    else if (delta) LEB_REC3(NV_, true, false)            \
    else if (row_decay) LEB_REC3(NV_, false, true)        \
    else LEB_REC3(NV_, false, false)                      \
  }
  if (nv == 1) LEB_REC2(1)
  else if (nv == 2) LEB_REC2(2)
  else if (nv == 4) LEB_REC2(4)
  else LEB_REC2(8)
#undef LEB_REC2
#undef LEB_REC3
  LEB_CHECK_LAUNCH("leb_gated_recurrence");
  return 0;
}

// What a row of the delta-rule mixer needs between its convolutions and its recurrence, one block a row:
//   q, k: silu, then unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times q_scale
//   v: silu;  write = sigmoid(b);  decay = exp(-exp(A_log_h) softplus(a + dt_bias)) per head and key channel
// qk [M, 2*Gk*d + H*e] is the convolution's output (q | k | v), `a` [M, H*d] the decay's pre-activation and
// `b` [M, H] the write strength's (row strides lda, ldb).  Results: qn, kn [M, Gk*d], vs [M, H*e], g [M, H*d], wr [M, H].
// A row's work is spread over blockIdx.y: first blocks of four heads of q | k (a warp a head), then blocks of
// DPREP_CHUNK numbers of v | decay | write, so that a decode step of a few rows still fills the machine.
constexpr int DPREP_CHUNK = 512;
__global__ void __launch_bounds__(128)
delta_prep_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vs, float* __restrict__ g,
                  float* __restrict__ wr, const float* __restrict__ qkv, int ldq, const float* __restrict__ a, int lda,
                  const float* __restrict__ bw, int ldb, const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                  int H, int Gk, int d, int e, float unit_eps, float q_scale) {
  pdl_wait();
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* row = qkv + m * ldq;
  const int head_blocks = (2 * Gk + nw - 1) / nw;
  if ((int)blockIdx.y < head_blocks) {      // heads of q, then heads of k
    const int hh = blockIdx.y * nw + warp;
    if (hh >= 2 * Gk) return;
    const float* src = row + (size_t)hh * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float x = silu_f(src[i]);
      ss += x * x;
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss + unit_eps) * (hh < Gk ? q_scale : 1.0f);
    float* dst = hh < Gk ? qn + m * (size_t)(Gk * d) + (size_t)hh * d : kn + m * (size_t)(Gk * d) + (size_t)(hh - Gk) * d;
    for (int i = lane; i < d; i += 32) dst[i] = silu_f(src[i]) * r;
    return;
  }
  const float* vrow = row + (size_t)2 * Gk * d;
  const int nv = H * e, ng = H * d;
  const int lo = ((int)blockIdx.y - head_blocks) * DPREP_CHUNK, hi = min(lo + DPREP_CHUNK, nv + ng + H);
  for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) {
    if (j < nv) {
      vs[m * (size_t)nv + j] = silu_f(vrow[j]);
    } else if (j < nv + ng) {
      const int i = j - nv;
      const float rate = expf(A_log[i / d]);
      g[m * (size_t)ng + i] = expf(-rate * softplus_f(a[m * lda + i] + dt_bias[i]));
    } else {
      const int i = j - nv - ng;
      wr[m * H + i] = sigmoid_f(bw[m * ldb + i]);
    }
  }
}

LEB_API int leb_delta_prep(float* qn, float* kn, float* vs, float* g, float* wr, const float* qkv, int ldq, const float* a,
                           int lda, const float* bw, int ldb, const float* dt_bias, const float* A_log, int M, int H, int Gk,
                           int d, int e, float unit_eps, float q_scale, cudaStream_t st) {
  if (M <= 0) return 0;
  LebPlainLaunches plain(true);
  const int blocks_y = ceil_div(2 * Gk, 4) + ceil_div(H * e + H * d + H, DPREP_CHUNK);
  LEB_REQUIRE(blocks_y <= 65535, "leb_delta_prep: a row of %d blocks", blocks_y);
  leb_launch(delta_prep_kernel, dim3(M, blocks_y), dim3(128), 0, st, qn, kn, vs, g, wr, qkv, ldq, a, lda, bw, ldb, dt_bias,
             A_log, H, Gk, d, e, unit_eps, q_scale);
  LEB_CHECK_LAUNCH("leb_delta_prep");
  return 0;
}

// What a row of the state-space mixer needs between its convolution and its recurrence:
//   xbc <- silu(xbc + conv_bias) in place over the C convolved channels;
//   dt = softplus(dt_raw + dt_bias) and decay = exp(-exp(A_log_h) dt), both [M, H].
__global__ void __launch_bounds__(128)
ssm_prep_kernel(float* __restrict__ xbc, int ldx, int C, const float* __restrict__ conv_bias, float* __restrict__ dt,
                float* __restrict__ decay, const float* __restrict__ dt_raw, int ldt, const float* __restrict__ dt_bias,
                const float* __restrict__ A_log, int H) {
  pdl_wait();
  const size_t m = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < C; i += gridDim.y * blockDim.x) {
    const float x = xbc[m * ldx + i] + (conv_bias ? conv_bias[i] : 0.f);
    xbc[m * ldx + i] = silu_f(x);
  }
  if (blockIdx.y != 0) return;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float t = softplus_f(dt_raw[m * ldt + i] + dt_bias[i]);
    dt[m * H + i] = t;
    decay[m * H + i] = expf(-expf(A_log[i]) * t);
  }
}

LEB_API int leb_ssm_prep(float* xbc, int ldx, int C, const float* conv_bias, float* dt, float* decay, const float* dt_raw,
                         int ldt, const float* dt_bias, const float* A_log, int M, int H, cudaStream_t st) {
  if (M <= 0) return 0;
  LebPlainLaunches plain(true);
  const int blocks_y = min(ceil_div(C, 4 * 128), 64);      // a thread takes about four channels
  leb_launch(ssm_prep_kernel, dim3(M, blocks_y), dim3(128), 0, st, xbc, ldx, C, conv_bias, dt, decay, dt_raw, ldt, dt_bias,
             A_log, H);
  LEB_CHECK_LAUNCH("leb_ssm_prep");
  return 0;
}

// A recurrent mixer's result on its way to the output projection: groups of `gs` neighbouring numbers of a
// row are divided by their root mean square (eps inside the root) and multiplied by a weight
// (w[j % wlen]: one weight for every group, or one per column), and the row is gated by a second
// row z: sigmoid(z) after the norm (gate_first = 0), or silu(z) before it (gate_first = 1).
// y, z float; out in the activation type.  A team takes a group: a warp (four groups a block, blockIdx.y counts
// blocks of groups), or for groups wider than GNG_WARP_MAX the whole block (blockIdx.y is the group).
constexpr int GNG_WARP_MAX = 256;
template <typename T>
__global__ void __launch_bounds__(128)
group_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ y, const float* __restrict__ z, int ldz,
                       const float* __restrict__ w, int C, int gs, int wlen, float eps, int gate_first) {
  __shared__ float red[4];
  pdl_wait();
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const bool wide = gs > GNG_WARP_MAX;
  const int gidx = wide ? blockIdx.y : blockIdx.y * nw + warp;
  const int t0 = wide ? threadIdx.x : lane, nt = wide ? blockDim.x : 32;
  const bool live = gidx < C / gs;     // only a warp-sized team can be idle: no block-wide wait follows for it
  const float* yr = y + m * C + (size_t)gidx * gs;
  const float* zr = z + m * ldz + (size_t)gidx * gs;
  float ss = 0.f;
  if (live)
    for (int i = t0; i < gs; i += nt) {
      const float x = gate_first ? yr[i] * silu_f(zr[i]) : yr[i];
      ss += x * x;
    }
  ss = warp_sum(ss);
  if (wide) {
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.f;
    for (int i = 0; i < nw; i++) ss += red[i];     // the same order in every thread
  }
  if (!live) return;
  const float r = 1.0f / sqrtf(ss / (float)gs + eps);
  for (int i = t0; i < gs; i += nt) {
    const int j = gidx * gs + i;
    const float x = gate_first ? yr[i] * silu_f(zr[i]) : yr[i];
    float val = x * r * w[j % wlen];
    if (!gate_first) val *= sigmoid_f(zr[i]);
    out[m * C + j] = from_f32<T>(val);
  }
}

LEB_API int leb_group_norm_gate(void* out, int dtype, const float* y, const float* z, int ldz, const float* w, int M, int C,
                                int gs, int wlen, float eps, int gate_first, cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(gs >= 1 && C % gs == 0 && wlen >= 1, "leb_group_norm_gate: %d columns in groups of %d", C, gs);
  LebPlainLaunches plain(true);
  const int groups = C / gs;
  const dim3 grid(M, gs > GNG_WARP_MAX ? groups : ceil_div(groups, 4));
  LEB_REQUIRE(grid.y <= 65535, "leb_group_norm_gate: %d groups in a row", groups);
  if (dtype == LEB_F32)
    leb_launch(group_norm_gate_kernel<float>, grid, dim3(128), 0, st, (float*)out, y, z, ldz, w, C, gs, wlen, eps, gate_first);
  else if (dtype == LEB_BF16)
    leb_launch(group_norm_gate_kernel<bf16>, grid, dim3(128), 0, st, (bf16*)out, y, z, ldz, w, C, gs, wlen, eps, gate_first);
  else
    return leb_fail("leb_group_norm_gate: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_group_norm_gate");
  return 0;
}

// ---- the post-norm layer arrangement and the embedding with learned positions ---------------------------
// x <- LN(alpha x + y) with weight and bias (variance = mean of the squared deviations), one block a row;
// with h, the same launch leaves the new row there in the activation type (the next sublayer's input).
template <typename TH>
__global__ void __launch_bounds__(512)
postnorm_residual_kernel(float* __restrict__ x, const float* __restrict__ y, float alpha, const float* __restrict__ w,
                         const float* __restrict__ bias, float eps, TH* __restrict__ h, int D, int vec) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[33];
  pdl_wait();
  const size_t m = blockIdx.x;
  float s = 0.f;
  if (vec) {      // D is a multiple of four and the rows start on 16 bytes: four numbers a load and a store
    const float4* x4 = reinterpret_cast<const float4*>(x + m * D);
    const float4* y4 = reinterpret_cast<const float4*>(y + m * D);
    float4* row4 = reinterpret_cast<float4*>(row);
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
      const float4 a = x4[i], c = y4[i];
      const float4 t = make_float4(alpha * a.x + c.x, alpha * a.y + c.y, alpha * a.z + c.z, alpha * a.w + c.w);
      row4[i] = t;
      s += (t.x + t.y) + (t.z + t.w);
    }
    const float mean = block_sum(s, red) / (float)D;
    float q = 0.f;
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
      const float4 t = row4[i];
      const float d0 = t.x - mean, d1 = t.y - mean, d2 = t.z - mean, d3 = t.w - mean;
      q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
    const float r = 1.0f / sqrtf(block_sum(q, red) / (float)D + eps);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
    float4* xo = reinterpret_cast<float4*>(x + m * D);
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
      const float4 t = row4[i], ww = w4[i], bb = bias ? b4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 o = make_float4((t.x - mean) * r * ww.x + bb.x, (t.y - mean) * r * ww.y + bb.y,
                                   (t.z - mean) * r * ww.z + bb.z, (t.w - mean) * r * ww.w + bb.w);
      xo[i] = o;
      if (h) {
        TH* hp = h + m * D + 4 * (size_t)i;
        hp[0] = from_f32<TH>(o.x);
        hp[1] = from_f32<TH>(o.y);
        hp[2] = from_f32<TH>(o.z);
        hp[3] = from_f32<TH>(o.w);
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float t = alpha * x[m * D + i] + y[m * D + i];
    row[i] = t;
    s += t;
  }
  const float mean = block_sum(s, red) / (float)D;
  float q = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float dlt = row[i] - mean;
    q += dlt * dlt;
  }
  const float r = 1.0f / sqrtf(block_sum(q, red) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float t = (row[i] - mean) * r * w[i] + (bias ? bias[i] : 0.f);
    x[m * D + i] = t;
    if (h) h[m * D + i] = from_f32<TH>(t);
  }
}

LEB_API int leb_postnorm_residual(float* x, const float* y, float alpha, const float* w, const float* bias, float eps,
                                  void* h, int h_dtype, int M, int D, cudaStream_t st) {
  if (M <= 0 || D <= 0) return 0;
  LEB_REQUIRE((size_t)D * sizeof(float) <= 160 * 1024, "leb_postnorm_residual: a width of %d does not fit shared memory", D);
  const size_t smem = (size_t)D * sizeof(float);
  const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
  const int vec = D % 4 == 0 && ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)bias) & 15) == 0);
  LebPlainLaunches plain(true);
  static bool set = false;
  if (smem > 48 * 1024 && !set) {
    cudaFuncSetAttribute(postnorm_residual_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    cudaFuncSetAttribute(postnorm_residual_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    set = true;
  }
  if (!h || h_dtype == LEB_F32)
    leb_launch(postnorm_residual_kernel<float>, dim3(M), dim3(threads), smem, st, x, y, alpha, w, bias, eps, (float*)h, D, vec);
  else if (h_dtype == LEB_BF16)
    leb_launch(postnorm_residual_kernel<bf16>, dim3(M), dim3(threads), smem, st, x, y, alpha, w, bias, eps, (bf16*)h, D, vec);
  else
    return leb_fail("leb_postnorm_residual: unknown dtype %d", h_dtype);
  LEB_CHECK_LAUNCH("leb_postnorm_residual");
  return 0;
}

// out[r] = LN(x[rows[r]]) * w + bias (rows null: the rows as they come); x float, out any activation type.
template <typename T>
__global__ void __launch_bounds__(512)
layernorm_bias_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                      const float* __restrict__ bias, const int* __restrict__ rows, int D, float eps) {
  __shared__ float red[33];
  pdl_wait();
  const size_t m = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[m] : m) * D;
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) s += xr[i];
  const float mean = block_sum(s, red) / (float)D;
  float q = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float dlt = xr[i] - mean;
    q += dlt * dlt;
  }
  const float r = 1.0f / sqrtf(block_sum(q, red) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    out[m * D + i] = from_f32<T>((xr[i] - mean) * r * w[i] + (bias ? bias[i] : 0.f));
}

LEB_API int leb_layernorm_bias(void* out, int dtype, const float* x, const float* w, const float* bias, const int* rows,
                               int M, int D, float eps, cudaStream_t st) {
  if (M <= 0 || D <= 0) return 0;
  const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
  LebPlainLaunches plain(true);
  if (dtype == LEB_F32)
    leb_launch(layernorm_bias_kernel<float>, dim3(M), dim3(threads), 0, st, (float*)out, x, w, bias, rows, D, eps);
  else if (dtype == LEB_BF16)
    leb_launch(layernorm_bias_kernel<bf16>, dim3(M), dim3(threads), 0, st, (bf16*)out, x, w, bias, rows, D, eps);
  else
    return leb_fail("leb_layernorm_bias: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_layernorm_bias");
  return 0;
}

// x[m] = table[token[m]] * scale + positions[row_pos[m]] as float; with h, the row in the activation type too.
template <typename T, typename TH>
__global__ void __launch_bounds__(256)
embed_positions_kernel(float* __restrict__ x, TH* __restrict__ h, const T* __restrict__ table, const int* __restrict__ tokens,
                       const float* __restrict__ positions, const int* __restrict__ row_pos, int D, int V, int n_pos,
                       float scale) {
  pdl_wait();
  const size_t m = blockIdx.x;
  int tok = tokens[m];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  int p = row_pos[m];
  p = p < 0 ? 0 : (p >= n_pos ? n_pos - 1 : p);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float t = to_f32(table[(size_t)tok * D + i]) * scale + positions[(size_t)p * D + i];
    x[m * D + i] = t;
    if (h) h[m * D + i] = from_f32<TH>(t);
  }
}

LEB_API int leb_embed_positions(float* x, void* h, int h_dtype, const void* table, int dtype, const int* tokens,
                                const float* positions, const int* row_pos, int M, int D, int V, int n_pos, float scale,
                                cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(dtype == LEB_F32 || dtype == LEB_BF16, "leb_embed_positions: unknown dtype %d", dtype);
  LebPlainLaunches plain(true);
  const dim3 grid(M), block(256);
  if (dtype == LEB_F32)
    leb_launch(embed_positions_kernel<float, float>, grid, block, 0, st, x, (float*)h, (const float*)table, tokens, positions,
               row_pos, D, V, n_pos, scale);
  else if (!h || h_dtype == LEB_BF16)
    leb_launch(embed_positions_kernel<bf16, bf16>, grid, block, 0, st, x, (bf16*)h, (const bf16*)table, tokens, positions,
               row_pos, D, V, n_pos, scale);
  else
    leb_launch(embed_positions_kernel<bf16, float>, grid, block, 0, st, x, (float*)h, (const bf16*)table, tokens, positions,
               row_pos, D, V, n_pos, scale);
  LEB_CHECK_LAUNCH("leb_embed_positions");
  return 0;
}

// out[i] = cast(x[i]): the residual stream in the activation type, for a sublayer that reads the stream itself.
template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ out, const float* __restrict__ x, size_t n) {
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f32<T>(x[i]);
}

LEB_API int leb_cast_rows(void* out, int dtype, const float* x, size_t n, cudaStream_t st) {
  if (n == 0) return 0;
  LebPlainLaunches plain(true);
  const dim3 grid((unsigned)((n + 255) / 256)), block(256);
  if (dtype == LEB_F32) leb_launch(cast_rows_kernel<float>, grid, block, 0, st, (float*)out, x, n);
  else if (dtype == LEB_BF16) leb_launch(cast_rows_kernel<bf16>, grid, block, 0, st, (bf16*)out, x, n);
  else return leb_fail("leb_cast_rows: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_cast_rows");
  return 0;
}

// Recurrences that run along a sequence one number at a time, and the small kernels around the matrix
// memory with exponential gates.  Everything here is float: gates, their logarithms and exponentials, the
// running maximum and the states are 32-bit whatever the model's activation type is.
//
// leb_min_gru: per channel S_t = (1 - z_t) S_(t-1) + z_t c_t with z = sigmoid(pz + bz) and the candidate
//   c = u + 1/2 for u >= 0, sigmoid(u) below (u = px + bx); the row's result is S_t * silu(pg).  One state
//   number per channel and sequence.  A thread owns a channel of a sequence and walks the step's rows in order;
//   the rows' inputs are asked for a few rows ahead, so the walk waits on arithmetic, not on memory.
// leb_exp_gates: log input gate i = cap tanh((pi + bi) / cap), log forget gate f = logsigmoid(cap tanh((pf + bf) / cap));
//   running maximum m_t = max(f_t + m_(t-1), i_t) from the sequence's carried m (zero at its start);
//   decay a_t = exp(f_t + m_(t-1) - m_t), write strength b_t = exp(i_t - m_t).  The gates of all rows are formed
//   side by side, the maximum walks the rows, the exponentials are again side by side.
// leb_exp_gates_finish: a head's read-out y [e] with its normaliser n.q in column e, both still without the
//   query's scale s: o = s y / (max(|s n.q|, exp(-m_t)) + 1e-6); o over its root mean square (eps inside the
//   root), times a weight over all heads' columns, times sigmoid(gate).
#include "common.cuh"

__device__ __forceinline__ float gs_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float gs_log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

constexpr int GRU_AHEAD = 4;      // rows whose inputs are in flight while one is computed

template <typename TO>
__global__ void __launch_bounds__(128)
min_gru_kernel(TO* __restrict__ out, const float* __restrict__ pz, const float* __restrict__ px, const float* __restrict__ pg,
               int ldp, const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
               const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen, int W) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int b = blockIdx.y;
  const int slot = seq_slot[b];
  const int n = seq_qlen ? seq_qlen[b] : 1;
  const size_t m0 = seq_qstart[b];
  const float zb = bz ? bz[c] : 0.f, xb = bx ? bx[c] : 0.f;
  float S = slot >= 0 ? state[(size_t)slot * W + c] : 0.f;
  float rz[GRU_AHEAD], rx[GRU_AHEAD], rg[GRU_AHEAD];
#pragma unroll
  for (int a = 0; a < GRU_AHEAD; a++)
    if (a < n) {
      rz[a] = pz[(m0 + a) * ldp + c];
      rx[a] = px[(m0 + a) * ldp + c];
      rg[a] = pg[(m0 + a) * ldp + c];
    }
  for (int t0 = 0; t0 < n; t0 += GRU_AHEAD) {
#pragma unroll
    for (int a = 0; a < GRU_AHEAD; a++) {
      const int t = t0 + a;
      if (t >= n) break;
      const float zr = rz[a], u = rx[a] + xb, g = rg[a];
      if (t + GRU_AHEAD < n) {
        rz[a] = pz[(m0 + t + GRU_AHEAD) * ldp + c];
        rx[a] = px[(m0 + t + GRU_AHEAD) * ldp + c];
        rg[a] = pg[(m0 + t + GRU_AHEAD) * ldp + c];
      }
      const float z = gs_sigmoid(zr + zb);
      const float cand = u >= 0.f ? u + 0.5f : gs_sigmoid(u);
      S = (1.0f - z) * S + z * cand;
      out[(m0 + t) * W + c] = from_f32<TO>(S * (g / (1.0f + expf(-g))));
    }
  }
  if (slot >= 0) state[(size_t)slot * W + c] = S;
}

// Long prompts: the rows of a sequence are cut into pieces of GRU_PIECE rows that run side by side.  The
// recurrence S_t = a_t S_(t-1) + b_t (a = 1 - z, b = z c) of a piece, started from zero, gives the piece's two
// numbers A = prod a_t and B = its last S; a piece's true start is the state carried in through the pieces before
// it, S_in(p) = A(p-1) S_in(p-1) + B(p-1), a short walk that every thread of the second launch does for itself.
constexpr int GRU_PIECE = 32;

__global__ void __launch_bounds__(128)
min_gru_pieces_kernel(float* __restrict__ sumA, float* __restrict__ sumB, const float* __restrict__ pz,
                      const float* __restrict__ px, int ldp, const float* __restrict__ bz, const float* __restrict__ bx,
                      const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen, int W, int max_pieces) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int p = blockIdx.y, b = blockIdx.z;
  const int n = seq_qlen[b];
  const int t0 = p * GRU_PIECE;
  if (t0 >= n) return;
  const int rows = min(GRU_PIECE, n - t0);
  const size_t m0 = (size_t)seq_qstart[b] + t0;
  const float zb = bz ? bz[c] : 0.f, xb = bx ? bx[c] : 0.f;
  float A = 1.f, S = 0.f;
#pragma unroll 8
  for (int t = 0; t < rows; t++) {
    const float z = gs_sigmoid(pz[(m0 + t) * ldp + c] + zb);
    const float u = px[(m0 + t) * ldp + c] + xb;
    const float cand = u >= 0.f ? u + 0.5f : gs_sigmoid(u);
    A *= 1.0f - z;
    S = (1.0f - z) * S + z * cand;
  }
  sumA[((size_t)b * max_pieces + p) * W + c] = A;
  sumB[((size_t)b * max_pieces + p) * W + c] = S;
}

template <typename TO>
__global__ void __launch_bounds__(128)
min_gru_finish_kernel(TO* __restrict__ out, const float* __restrict__ sumA, float* sumB,
                      const float* __restrict__ pz, const float* __restrict__ px, const float* __restrict__ pg, int ldp,
                      const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
                      const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                      int W, int max_pieces) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int p = blockIdx.y, b = blockIdx.z;
  const int n = seq_qlen[b];
  const int t0 = p * GRU_PIECE;
  if (t0 >= n) return;
  const int rows = min(GRU_PIECE, n - t0);
  const int slot = seq_slot[b];
  const size_t m0 = (size_t)seq_qstart[b] + t0;
  const float zb = bz ? bz[c] : 0.f, xb = bx ? bx[c] : 0.f;
  float S = slot >= 0 ? state[(size_t)slot * W + c] : 0.f;
  for (int q = 0; q < p; q++) {
    const size_t at = ((size_t)b * max_pieces + q) * W + c;
    S = sumA[at] * S + sumB[at];
  }
#pragma unroll 8
  for (int t = 0; t < rows; t++) {
    const float z = gs_sigmoid(pz[(m0 + t) * ldp + c] + zb);
    const float u = px[(m0 + t) * ldp + c] + xb;
    const float g = pg[(m0 + t) * ldp + c];
    const float cand = u >= 0.f ? u + 0.5f : gs_sigmoid(u);
    S = (1.0f - z) * S + z * cand;
    out[(m0 + t) * W + c] = from_f32<TO>(S * (g / (1.0f + expf(-g))));
  }
  // The piece that holds the sequence's last row leaves the state.  Every piece read the carried state above, and
  // the write must not pass those reads: the pieces of a sequence are blocks of one launch that may run in any
  // order, so the new state goes to the scratch row of this piece and a third, tiny launch stores it.
  if (t0 + rows == n) sumB[((size_t)b * max_pieces + p) * W + c] = S;
}

__global__ void __launch_bounds__(128)
min_gru_state_kernel(float* __restrict__ state, const float* __restrict__ sumB, const int* __restrict__ seq_slot,
                     const int* __restrict__ seq_qlen, int W, int max_pieces) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  const int slot = seq_slot[b], n = seq_qlen[b];
  if (c >= W || slot < 0 || n <= 0) return;
  const int last = (n - 1) / GRU_PIECE;
  state[(size_t)slot * W + c] = sumB[((size_t)b * max_pieces + last) * W + c];
}

LEB_API int leb_min_gru_piece_rows() { return GRU_PIECE; }

// out [M, W] in the activation type; pz, px, pg float with one row stride (column ranges of one projection);
// bz, bx [W] or null; state [slots][W]; seq_qlen null: one row per sequence.
// scratch: null, or 2 * B * ceil(max_qlen / leb_min_gru_piece_rows()) * W floats: the rows of long sequences then
// run in pieces side by side (three launches).
LEB_API int leb_min_gru(void* out, int dtype, const float* pz, const float* px, const float* pg, int ldp, const float* bz,
                        const float* bx, float* state, const int* seq_slot, const int* seq_qstart, const int* seq_qlen,
                        int B, int W, int max_qlen, float* scratch, cudaStream_t st) {
  if (B <= 0 || W <= 0) return 0;
  LEB_REQUIRE(B <= 65535, "leb_min_gru: step too large");
  LEB_REQUIRE(dtype == LEB_F32 || dtype == LEB_BF16, "leb_min_gru: unknown dtype %d", dtype);
  LebPlainLaunches plain(true);
  if (scratch && seq_qlen && max_qlen > GRU_PIECE) {
    const int pieces = ceil_div(max_qlen, GRU_PIECE);
    LEB_REQUIRE(pieces <= 65535, "leb_min_gru: step too large");
    float* sumA = scratch;
    float* sumB = scratch + (size_t)B * pieces * W;
    const dim3 grid(ceil_div(W, 128), pieces, B), block(128);
    leb_launch(min_gru_pieces_kernel, grid, block, 0, st, sumA, sumB, pz, px, ldp, bz, bx, seq_qstart, seq_qlen, W, pieces);
    LEB_CHECK_LAUNCH("leb_min_gru (pieces)");
    if (dtype == LEB_F32)
      leb_launch(min_gru_finish_kernel<float>, grid, block, 0, st, (float*)out, sumA, sumB, pz, px, pg, ldp, bz, bx, state,
                 seq_slot, seq_qstart, seq_qlen, W, pieces);
    else
      leb_launch(min_gru_finish_kernel<bf16>, grid, block, 0, st, (bf16*)out, sumA, sumB, pz, px, pg, ldp, bz, bx, state,
                 seq_slot, seq_qstart, seq_qlen, W, pieces);
    LEB_CHECK_LAUNCH("leb_min_gru (finish)");
    leb_launch(min_gru_state_kernel, dim3(ceil_div(W, 128), B), block, 0, st, state, sumB, seq_slot, seq_qlen, W, pieces);
    LEB_CHECK_LAUNCH("leb_min_gru (state)");
    return 0;
  }
  const dim3 grid(ceil_div(W, 128), B), block(128);
  if (dtype == LEB_F32)
    leb_launch(min_gru_kernel<float>, grid, block, 0, st, (float*)out, pz, px, pg, ldp, bz, bx, state, seq_slot, seq_qstart,
               seq_qlen, W);
  else if (dtype == LEB_BF16)
    leb_launch(min_gru_kernel<bf16>, grid, block, 0, st, (bf16*)out, pz, px, pg, ldp, bz, bx, state, seq_slot, seq_qstart,
               seq_qlen, W);
  else
    return leb_fail("leb_min_gru: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_min_gru");
  return 0;
}

// The gates of all rows side by side (first launch): write <- i, decay <- f.
__global__ void __launch_bounds__(256)
exp_gates_rows_kernel(float* __restrict__ decay, float* __restrict__ write, const float* __restrict__ pi,
                      const float* __restrict__ pf, int ldp, const float* __restrict__ bi, const float* __restrict__ bf,
                      float cap, int H, size_t total) {
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t m = idx / H;
  const int h = (int)(idx - m * H);
  const float ri = pi[m * ldp + h] + (bi ? bi[h] : 0.f);
  const float rf = pf[m * ldp + h] + (bf ? bf[h] : 0.f);
  write[idx] = cap * tanhf(ri / cap);
  decay[idx] = gs_log_sigmoid(cap * tanhf(rf / cap));
}

// Second launch: a block takes a sequence and walks its rows in pieces that fit shared memory: the piece's f and i
// come in side by side, the maximum walks the piece there (one thread a head, an addition and a maximum per row,
// no trip to global memory inside the walk), and the exponentials are again formed side by side.
constexpr int EXG_FLOATS = 3 * 4096;      // shared floats of a block: f, i and m of a piece
__global__ void __launch_bounds__(1024)
exp_gates_kernel(float* __restrict__ decay, float* __restrict__ write, float* __restrict__ mrow,
                 float* __restrict__ mstate, const int* __restrict__ seq_slot, const int* __restrict__ seq_qstart,
                 const int* __restrict__ seq_qlen, int H, int piece, const float* __restrict__ pi,
                 const float* __restrict__ pf, int ldp, const float* __restrict__ bi, const float* __restrict__ bf, float cap) {
  __shared__ float sm[EXG_FLOATS];
  pdl_wait();
  const int b = blockIdx.x;
  const int slot = seq_slot[b];
  const int n = seq_qlen ? seq_qlen[b] : 1;
  const size_t m0 = seq_qstart[b];
  float* fs = sm;                       // [piece][H]
  float* is = sm + (size_t)piece * H;
  float* ms = is + (size_t)piece * H;   // [piece + 1][H]: row 0 holds the maximum before the piece
  for (int h = threadIdx.x; h < H; h += blockDim.x) ms[h] = slot >= 0 ? mstate[(size_t)slot * H + h] : 0.f;
  for (int t0 = 0; t0 < n; t0 += piece) {
    const int rows = min(piece, n - t0);
    for (int idx = threadIdx.x; idx < rows * H; idx += blockDim.x) {
      if (pi) {      // a step of few rows: the gates are formed here, in the one launch
        const int t = idx / H, h = idx - t * H;
        const float ri = pi[(m0 + t0 + t) * ldp + h] + (bi ? bi[h] : 0.f);
        const float rf = pf[(m0 + t0 + t) * ldp + h] + (bf ? bf[h] : 0.f);
        is[idx] = cap * tanhf(ri / cap);
        fs[idx] = gs_log_sigmoid(cap * tanhf(rf / cap));
      } else {
        const size_t at = (m0 + t0) * H + idx;
        fs[idx] = decay[at];
        is[idx] = write[at];
      }
    }
    __syncthreads();
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      float m = ms[h];
#pragma unroll 8
      for (int t = 0; t < rows; t++) {
        m = fmaxf(fs[t * H + h] + m, is[t * H + h]);
        ms[(t + 1) * H + h] = m;
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * H; idx += blockDim.x) {
      const float before = ms[idx], now = ms[idx + H];
      const size_t at = (m0 + t0) * H + idx;
      decay[at] = expf(fs[idx] + before - now);
      write[at] = expf(is[idx] - now);
      mrow[at] = now;
    }
    __syncthreads();
    for (int h = threadIdx.x; h < H; h += blockDim.x) ms[h] = ms[rows * H + h];      // each thread its own heads: no race
  }
  __syncthreads();
  if (slot >= 0 && n > 0)
    for (int h = threadIdx.x; h < H; h += blockDim.x) mstate[(size_t)slot * H + h] = ms[h];
}

// decay, write, mrow [M, H] float; pi, pf float with one row stride; bi, bf [H] or null; mstate [slots][H].
LEB_API int leb_exp_gates(float* decay, float* write, float* mrow, const float* pi, const float* pf, int ldp, const float* bi,
                          const float* bf, float cap, float* mstate, const int* seq_slot, const int* seq_qstart,
                          const int* seq_qlen, int M, int B, int H, cudaStream_t st) {
  if (B <= 0 || H <= 0 || M <= 0) return 0;
  LEB_REQUIRE(cap > 0.f, "leb_exp_gates: the gates' cap must be positive, got %g", (double)cap);
  LEB_REQUIRE(H <= 2048, "leb_exp_gates: %d heads (up to 2048)", H);
  LebPlainLaunches plain(true);
  const int piece = min(256, (EXG_FLOATS / 3 - H) / H);      // rows of a piece: f, i and m (one row more) fit
  const bool few = M <= 4 * B;      // decode steps and the like: one launch forms the gates and walks them
  if (!few) {
    const size_t total = (size_t)M * H;
    leb_launch(exp_gates_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, decay, write, pi, pf, ldp, bi,
               bf, cap, H, total);
    LEB_CHECK_LAUNCH("leb_exp_gates (rows)");
  }
  // many threads where a sequence brings many rows: the pieces' loads and exponentials are what takes the time
  leb_launch(exp_gates_kernel, dim3(B), dim3(few ? 128 : 1024), 0, st, decay, write, mrow, mstate, seq_slot, seq_qstart,
             seq_qlen, H, piece, few ? pi : nullptr, pf, ldp, bi, bf, cap);
  LEB_CHECK_LAUNCH("leb_exp_gates");
  return 0;
}

// A warp takes a (row, head): y [M, H (e + 1)] with the normaliser's product in a head's last column.
template <typename TO>
__global__ void __launch_bounds__(128)
exp_gates_finish_kernel(TO* __restrict__ out, const float* __restrict__ y, const float* __restrict__ mrow,
                        const float* __restrict__ gate, int ldg, const float* __restrict__ w, float qscale, float eps, int M,
                        int H, int e) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t pair = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= (size_t)M * H) return;
  const size_t m = pair / H;
  const int h = (int)(pair - m * H);
  const float* yr = y + (m * H + h) * (size_t)(e + 1);
  const float den = fmaxf(fabsf(qscale * yr[e]), expf(-mrow[m * H + h])) + 1e-6f;
  float ss = 0.f;
  for (int i = lane; i < e; i += 32) {
    const float o = qscale * yr[i] / den;
    ss += o * o;
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)e + eps);
  for (int i = lane; i < e; i += 32) {
    const float o = qscale * yr[i] / den;
    const float g = gate[m * ldg + (size_t)h * e + i];
    out[(m * H + h) * (size_t)e + i] = from_f32<TO>(o * r * w[(size_t)h * e + i] * gs_sigmoid(g));
  }
}

LEB_API int leb_exp_gates_finish(void* out, int dtype, const float* y, const float* mrow, const float* gate, int ldg,
                                 const float* w, float qscale, float eps, int M, int H, int e, cudaStream_t st) {
  if (M <= 0 || H <= 0 || e <= 0) return 0;
  LebPlainLaunches plain(true);
  const size_t pairs = (size_t)M * H;
  const dim3 grid((unsigned)((pairs + 3) / 4)), block(128);
  if (dtype == LEB_F32)
    leb_launch(exp_gates_finish_kernel<float>, grid, block, 0, st, (float*)out, y, mrow, gate, ldg, w, qscale, eps, M, H, e);
  else if (dtype == LEB_BF16)
    leb_launch(exp_gates_finish_kernel<bf16>, grid, block, 0, st, (bf16*)out, y, mrow, gate, ldg, w, qscale, eps, M, H, e);
  else
    return leb_fail("leb_exp_gates_finish: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_exp_gates_finish");
  return 0;
}

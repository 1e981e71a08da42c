// Recurrent mixers: a linear recurrence with a diagonal decay over a matrix state per head,
//   S_t = diag(a_t) S_{t-1} + k_t v_t^T        (S is K x V; a_t a vector over K, or one number)
//   o_t = S_t^T q_t,
// the short causal convolution that some of them put in front of it, and the gated group norm
// that follows it.  Gated linear attention (a decay per key channel) and state-space mixers of
// the Mamba-2 kind (a scalar decay per head, keys and queries shared by the heads of a group,
// values scaled by the step size) are both this recurrence; which one runs is data.  So is the
// gated delta rule, whose write is the error of the state's own answer for the key:
//   S <- diag(a_t) S;  u = b_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t.
//
// Everything here is 32-bit: the inputs are the 32-bit results of the projections, the state
// lives in 32-bit floats in the request's state slot, decays and step sizes are made here from
// the projected values.  The tokens of a request are visited one after the other and every sum
// has a fixed order, so the result for a token is the same bits however the prompt was cut into
// steps and whatever else is in the batch.
//
// Which rows of a step belong to which request is read on the device: either every row is a
// request of its own (`single`: slot = row_slot[row]), or a table of (first row, end row) per
// request slot made by llm_segment_table from row_slot (with the list of the slots that have rows).  No host data is involved, so steps of
// single tokens can be recorded and replayed.
#include "common.cuh"

namespace {

// The table has three integers per request slot s: (first row, row after the last) of the rows
// whose request slot is s, (0, 0) for none; and, as the third of entry i, the slot of the i-th
// request that has rows in this step (in no particular order), so that a kernel can run one
// block per request of the step instead of one per slot.  The rows of a request are consecutive.
constexpr int SEG = 3;
__global__ void segment_table_kernel(const int* __restrict__ row_slot, int rows, int* __restrict__ seg,
                                     int n_slots) {
  __shared__ int count;
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) count = 0;
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) seg[SEG * s] = seg[SEG * s + 1] = 0, seg[SEG * s + 2] = -1;
  __syncthreads();
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    const int s = row_slot[r];
    if (s < 0 || s >= n_slots) continue;
    if (r == 0 || row_slot[r - 1] != s) {
      seg[SEG * s] = r;
      seg[SEG * atomicAdd(&count, 1) + 2] = s;
    }
    if (r == rows - 1 || row_slot[r + 1] != s) seg[SEG * s + 1] = r + 1;
  }
}

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

enum DecayKind : int {
  DECAY_VECTOR = 0,        // a = d                       d per (row, head, key channel)
  DECAY_SIGMOID_POW = 1,   // a = sigmoid(d)^c            d per (row, head, key channel), c a constant
  DECAY_RATE_STEP = 2,     // step = softplus(d + p1[h]); a = exp(-exp(p0[h]) * step); v is scaled by step
                           //                             d per (row, head)
  DECAY_SCALAR_INPUT = 3,  // a = d, v is scaled by d2    d, d2 per (row, head): a decay and an input
                           //                             weight that another kernel has made
};
// (With the delta rule DECAY_RATE_STEP leaves v as it is: the step only makes the decay.)

struct ScanArgs {
  const float* q; int q_stride;          // q[row * q_stride + g * K + i], g = h / (H / G)
  const float* k; int k_stride;          // k[row * k_stride + g * K + i]
  const float* v; int v_stride;          // v[row * v_stride + h * V + j]
  const float* d; int d_stride;          // the decay's argument (see DecayKind)
  const float* d2;                       // DECAY_SCALAR_INPUT: the input weight, strided as d
  int v_cols;                            // value channels of a head in v: V, or V - 1 when the last
                                         // state column is fed the constant 1 (`ones`)
  int ones;
  const float* p0; const float* p1;      // per-head constants of DECAY_RATE_STEP
  float c;                               // the exponent of DECAY_SIGMOID_POW
  float q_scale;                         // q is multiplied by it (applied to the head's output: the same product)
  float* state; long long state_stride;  // state[slot * state_stride + ((h * V) + j) * K + i]
  float* out; int out_stride;            // out[row * out_stride + h * V + j]
  const int* seg; const int* row_slot;
  int single, H, G, K, V, kind;
  // the delta rule: beta[row * beta_stride + h] is the write strength before its sigmoid;
  // `unit`: q and k of every head are divided by sqrt(sum of squares + unit_floor) first
  const float* beta; int beta_stride;
  int unit; float unit_floor;
  int tail_only;        // only the last (rows of the request) % 4 rows: the others went in groups of four
};

constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A block owns a tile of value channels of one head of one request and walks the request's
// tokens of the step in order.  L lanes share a group of four columns: lane i of the group holds,
// of each of the four, the state rows 4 (i + L n) + e (n < NF, e < 4) in registers, so one
// 16-byte read of q, k and the decay from shared memory serves sixteen state elements.  Per
// token a lane has four partial sums (one per column); they are summed over the L lanes by a
// butterfly whose first two steps each hand half of the columns to the partner, six shuffles
// for 32 lanes.  The tokens' q, k and decay arguments come into shared memory a chunk of tokens
// at a time by asynchronous copies, two chunks in flight: while one chunk is walked the next is
// on its way.
//
// DELTA: the gated delta rule.  Per token the state is decayed, its answers for the key and for
// the query are summed in one pass (two sets of partial sums), the write u = b (v - S^T k) is
// made where the key's sums end up, handed back to the L lanes of the group, and added as
// k u^T; the output is the decayed state's answer for the query plus u (k . q), which is what
// the written state answers.  q and k are made unit vectors (and q scaled) in shared memory once
// per token, with k . q beside them.
template <int L, int NF, bool VEC, bool DELTA>
__global__ void __launch_bounds__(SCAN_THREADS) linear_recurrence_kernel(const ScanArgs a) {
  constexpr int KP = 4 * L * NF;                            // key channels, padded
  constexpr int GROUPS = 32 / L;                            // column groups of a warp
  constexpr int COLS = 4 * GROUPS * (SCAN_THREADS / 32);    // value channels of a block
  constexpr int TC = KP >= 512 ? 2 : (KP >= 256 ? 4 : (KP >= 128 ? 8 : 16));  // tokens of a chunk
  __shared__ __align__(16) float q_s[2][TC][KP];
  __shared__ __align__(16) float k_s[2][TC][KP];
  __shared__ __align__(16) float a_s[2][VEC ? TC : 1][VEC ? KP : 4];
  __shared__ __align__(16) float v_s[2][TC][COLS];
  __shared__ float d_s[2][TC];          // scalar decay: its argument, then the decay itself
  __shared__ float w_s[2][TC];          // DECAY_SCALAR_INPUT: the input weight
  __shared__ float b_s[2][DELTA ? TC : 1];      // the delta rule: write strength, and k . q
  __shared__ float kq_s[2][DELTA ? TC : 1];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int slot, first, end;
  if (a.single) {
    first = blockIdx.x, end = first + 1, slot = a.row_slot[first];
  } else {
    slot = a.seg[SEG * blockIdx.x + 2];
    if (slot < 0) return;
    first = a.seg[SEG * slot], end = a.seg[SEG * slot + 1];
  }
  if (a.tail_only) first = end - ((end - first) & 3);
  if (end <= first) return;
  const int K = a.K, V = a.V, g = h / (a.H / a.G);
  const int j0 = blockIdx.z * COLS;
  const int li = lane % L;
  const int c0 = (warp * GROUPS + lane / L) * 4, jc = j0 + c0;     // this lane's four columns
  float* sbase = a.state + (size_t)slot * a.state_stride + (size_t)h * V * K;
  const bool k4 = (K & 3) == 0 && ((uintptr_t)sbase & 15) == 0;

  // key channels beyond K: they hold nothing and must stay that way
  for (int idx = tid; idx < 2 * TC * (KP - K); idx += SCAN_THREADS) {
    const int st = idx / (TC * (KP - K)), rem = idx - st * TC * (KP - K);
    const int tt = rem / (KP - K), i = K + rem - tt * (KP - K);
    q_s[st][tt][i] = 0.f;
    k_s[st][tt][i] = 0.f;
    if (VEC) a_s[st][tt][i] = 1.f;
  }
  // whether whole 16-byte pieces can be copied: every row of q, k and the decay's argument
  // starts on a 16-byte boundary
  const bool wide = (K & 3) == 0 && !((a.q_stride | a.k_stride | (VEC ? a.d_stride : 0)) & 3) &&
                    !(((uintptr_t)(a.q + g * K) | (uintptr_t)(a.k + g * K) |
                       (VEC ? (uintptr_t)(a.d + h * K) : 0)) & 15);
  auto fetch = [&](int st, int t0) {
    const int n_tok = min(TC, end - t0);
    if (wide) {
      const int k4n = K >> 2;
      for (int idx = tid; idx < n_tok * k4n; idx += SCAN_THREADS) {
        const int tt = idx / k4n, i = (idx - tt * k4n) << 2;
        const size_t row = (size_t)(t0 + tt);
        cp_async16(&q_s[st][tt][i], a.q + row * a.q_stride + g * K + i);
        cp_async16(&k_s[st][tt][i], a.k + row * a.k_stride + g * K + i);
        if (VEC) cp_async16(&a_s[st][tt][i], a.d + row * a.d_stride + h * K + i);
      }
    } else {
      for (int idx = tid; idx < n_tok * K; idx += SCAN_THREADS) {
        const int tt = idx / K, i = idx - tt * K;
        const size_t row = (size_t)(t0 + tt);
        cp_async4(&q_s[st][tt][i], a.q + row * a.q_stride + g * K + i);
        cp_async4(&k_s[st][tt][i], a.k + row * a.k_stride + g * K + i);
        if (VEC) cp_async4(&a_s[st][tt][i], a.d + row * a.d_stride + h * K + i);
      }
    }
    for (int idx = tid; idx < n_tok * COLS; idx += SCAN_THREADS) {
      const int tt = idx / COLS, cc = idx - tt * COLS;
      if (j0 + cc < a.v_cols)
        cp_async4(&v_s[st][tt][cc], a.v + (size_t)(t0 + tt) * a.v_stride + h * a.v_cols + j0 + cc);
      else
        v_s[st][tt][cc] = (a.ones && j0 + cc == V - 1) ? 1.f : 0.f;
    }
    if (!VEC)
      for (int tt = tid; tt < n_tok; tt += SCAN_THREADS) {
        cp_async4(&d_s[st][tt], a.d + (size_t)(t0 + tt) * a.d_stride + h);
        if (a.kind == DECAY_SCALAR_INPUT) cp_async4(&w_s[st][tt], a.d2 + (size_t)(t0 + tt) * a.d_stride + h);
      }
    if (DELTA)
      for (int tt = tid; tt < n_tok; tt += SCAN_THREADS)
        cp_async4(&b_s[st][tt], a.beta + (size_t)(t0 + tt) * a.beta_stride + h);
    cp_async_commit();
  };

  fetch(0, first);
  float s[NF][4][4];       // [n][row e][column c]
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const bool live = jc + c < V;
    const float* srow = sbase + (size_t)(live ? jc + c : 0) * K;
#pragma unroll
    for (int n = 0; n < NF; ++n) {
      const int i0 = 4 * (li + L * n);
      if (live && k4 && i0 + 3 < K) {
        const float4 t = *reinterpret_cast<const float4*>(srow + i0);
        s[n][0][c] = t.x, s[n][1][c] = t.y, s[n][2][c] = t.z, s[n][3][c] = t.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e][c] = (live && i0 + e < K) ? srow[i0 + e] : 0.f;
      }
    }
  }

  const float rate = a.kind == DECAY_RATE_STEP ? expf(a.p0[h]) : 0.f;
  const float bias = a.kind == DECAY_RATE_STEP ? a.p1[h] : 0.f;
  const float q_scale = a.q_scale;
  const bool up1 = (li & (L / 2)) != 0, up2 = (li & (L / 4)) != 0;
  const int my_col = jc + 2 * (up1 ? 1 : 0) + (up2 ? 1 : 0);
  const bool writer = (li & (L / 4 - 1)) == 0 && my_col < V;
  int st = 0;
  for (int t0 = first; t0 < end; t0 += TC, st ^= 1) {
    const int n_tok = min(TC, end - t0);
    if (t0 + TC < end) {
      fetch(st ^ 1, t0 + TC);       // (its stage was walked two chunks ago; a barrier lies between)
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // ---- the decay from its argument, once per token
    if (VEC) {
      if (a.kind == DECAY_SIGMOID_POW)
        for (int idx = tid; idx < n_tok * K; idx += SCAN_THREADS) {
          const int tt = idx / K, i = idx - tt * K;
          // sigmoid(d)^c = exp(c * log sigmoid(d)), log sigmoid(d) = -softplus(-d)
          a_s[st][tt][i] = expf(-a.c * softplus_f(-a_s[st][tt][i]));
        }
    } else if (a.kind == DECAY_SCALAR_INPUT) {
      for (int idx = tid; idx < n_tok * COLS; idx += SCAN_THREADS) {
        const int tt = idx / COLS, cc = idx - tt * COLS;
        v_s[st][tt][cc] *= w_s[st][tt];
      }
    } else {
      if (!DELTA) {
        for (int idx = tid; idx < n_tok * COLS; idx += SCAN_THREADS) {
          const int tt = idx / COLS, cc = idx - tt * COLS;
          v_s[st][tt][cc] *= softplus_f(d_s[st][tt] + bias);
        }
        __syncthreads();
      }
      for (int tt = tid; tt < n_tok; tt += SCAN_THREADS)
        d_s[st][tt] = expf(-rate * softplus_f(d_s[st][tt] + bias));
    }
    if (DELTA) {
      // a warp per token: unit vectors, the query's scale, k . q, the write strength
      for (int tt = warp; tt < n_tok; tt += SCAN_THREADS / 32) {
        float sq = 0.f, sk = 0.f;
        if (a.unit) {
          for (int i = lane; i < K; i += 32) {
            sq = fmaf(q_s[st][tt][i], q_s[st][tt][i], sq);
            sk = fmaf(k_s[st][tt][i], k_s[st][tt][i], sk);
          }
          sq = warp_sum(sq), sk = warp_sum(sk);
        }
        const float fq = (a.unit ? 1.0f / sqrtf(sq + a.unit_floor) : 1.f) * q_scale;
        const float fk = a.unit ? 1.0f / sqrtf(sk + a.unit_floor) : 1.f;
        float dot = 0.f;
        for (int i = lane; i < K; i += 32) {
          const float qv = q_s[st][tt][i] * fq, kv = k_s[st][tt][i] * fk;
          q_s[st][tt][i] = qv, k_s[st][tt][i] = kv;
          dot = fmaf(qv, kv, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) {
          kq_s[st][tt] = dot;
          b_s[st][tt] = 1.f / (1.f + expf(-b_s[st][tt]));
        }
      }
    }
    __syncthreads();
    // ---- the tokens of the chunk, one after the other
#pragma unroll 4
    for (int tt = 0; tt < n_tok; ++tt) {
      const float4 vv = *reinterpret_cast<const float4*>(&v_s[st][tt][c0]);
      const float a1 = VEC ? 1.f : d_s[st][tt];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (DELTA) {
        float ack[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int n = 0; n < NF; ++n) {
          const float4 qq = *reinterpret_cast<const float4*>(&q_s[st][tt][4 * (li + L * n)]);
          const float4 kk = *reinterpret_cast<const float4*>(&k_s[st][tt][4 * (li + L * n)]);
          float4 aa = make_float4(a1, a1, a1, a1);
          if (VEC) aa = *reinterpret_cast<const float4*>(&a_s[st][tt][4 * (li + L * n)]);
          const float qe[4] = {qq.x, qq.y, qq.z, qq.w}, ke[4] = {kk.x, kk.y, kk.z, kk.w};
          const float ae[4] = {aa.x, aa.y, aa.z, aa.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              s[n][e][c] *= ae[e];
              ack[c] = fmaf(s[n][e][c], ke[e], ack[c]);
              acc[c] = fmaf(s[n][e][c], qe[e], acc[c]);
            }
        }
        // both sets of sums over the L lanes of the group, as below
        const float rk0 = __shfl_xor_sync(0xffffffffu, up1 ? ack[0] : ack[2], L / 2);
        const float rk1 = __shfl_xor_sync(0xffffffffu, up1 ? ack[1] : ack[3], L / 2);
        const float rq0 = __shfl_xor_sync(0xffffffffu, up1 ? acc[0] : acc[2], L / 2);
        const float rq1 = __shfl_xor_sync(0xffffffffu, up1 ? acc[1] : acc[3], L / 2);
        const float bk0 = (up1 ? ack[2] : ack[0]) + rk0, bk1 = (up1 ? ack[3] : ack[1]) + rk1;
        const float bq0 = (up1 ? acc[2] : acc[0]) + rq0, bq1 = (up1 ? acc[3] : acc[1]) + rq1;
        float sumk = (up2 ? bk1 : bk0) + __shfl_xor_sync(0xffffffffu, up2 ? bk0 : bk1, L / 4);
        float sumq = (up2 ? bq1 : bq0) + __shfl_xor_sync(0xffffffffu, up2 ? bq0 : bq1, L / 4);
#pragma unroll
        for (int o = L / 8; o > 0; o >>= 1) {
          sumk += __shfl_xor_sync(0xffffffffu, sumk, o);
          sumq += __shfl_xor_sync(0xffffffffu, sumq, o);
        }
        // every lane now holds both sums of the column 2 up1 + up2 of its group
        const float v_mine = up1 ? (up2 ? vv.w : vv.z) : (up2 ? vv.y : vv.x);
        const float u_mine = b_s[st][tt] * (v_mine - sumk);
        if (writer) a.out[(size_t)(t0 + tt) * a.out_stride + h * V + my_col] = fmaf(u_mine, kq_s[st][tt], sumq);
        const int base = lane - li;
        const float ue[4] = {__shfl_sync(0xffffffffu, u_mine, base), __shfl_sync(0xffffffffu, u_mine, base + L / 4),
                             __shfl_sync(0xffffffffu, u_mine, base + L / 2),
                             __shfl_sync(0xffffffffu, u_mine, base + L / 2 + L / 4)};
#pragma unroll
        for (int n = 0; n < NF; ++n) {
          const float4 kk = *reinterpret_cast<const float4*>(&k_s[st][tt][4 * (li + L * n)]);
          const float ke[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[n][e][c] = fmaf(ke[e], ue[c], s[n][e][c]);
        }
        continue;
      }
#pragma unroll
      for (int n = 0; n < NF; ++n) {
        const float4 qq = *reinterpret_cast<const float4*>(&q_s[st][tt][4 * (li + L * n)]);
        const float4 kk = *reinterpret_cast<const float4*>(&k_s[st][tt][4 * (li + L * n)]);
        float4 aa = make_float4(a1, a1, a1, a1);
        if (VEC) aa = *reinterpret_cast<const float4*>(&a_s[st][tt][4 * (li + L * n)]);
        const float qe[4] = {qq.x, qq.y, qq.z, qq.w}, ke[4] = {kk.x, kk.y, kk.z, kk.w};
        const float ae[4] = {aa.x, aa.y, aa.z, aa.w}, ve[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            s[n][e][c] = fmaf(ae[e], s[n][e][c], ke[e] * ve[c]);
            acc[c] = fmaf(s[n][e][c], qe[e], acc[c]);
          }
      }
      // sum over the L lanes of the group: hand two columns to the partner, then one, then a
      // plain butterfly over what is left
      const float r0 = __shfl_xor_sync(0xffffffffu, up1 ? acc[0] : acc[2], L / 2);
      const float r1 = __shfl_xor_sync(0xffffffffu, up1 ? acc[1] : acc[3], L / 2);
      const float b0 = (up1 ? acc[2] : acc[0]) + r0, b1 = (up1 ? acc[3] : acc[1]) + r1;
      float sum = (up2 ? b1 : b0) + __shfl_xor_sync(0xffffffffu, up2 ? b0 : b1, L / 4);
#pragma unroll
      for (int o = L / 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (writer) a.out[(size_t)(t0 + tt) * a.out_stride + h * V + my_col] = sum * q_scale;
    }
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (jc + c >= V) continue;
    float* srow = sbase + (size_t)(jc + c) * K;
#pragma unroll
    for (int n = 0; n < NF; ++n) {
      const int i0 = 4 * (li + L * n);
      if (k4 && i0 + 3 < K) {
        *reinterpret_cast<float4*>(srow + i0) = make_float4(s[n][0][c], s[n][1][c], s[n][2][c], s[n][3][c]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (i0 + e < K) srow[i0 + e] = s[n][e][c];
      }
    }
  }
}

template <int L, int NF>
int launch_scan(const ScanArgs& a, int blocks_x, cudaStream_t stream) {
  constexpr int COLS = 4 * (32 / L) * (SCAN_THREADS / 32);
  const dim3 grid(blocks_x, a.H, (a.V + COLS - 1) / COLS);
  const bool scalar = a.kind == DECAY_RATE_STEP || a.kind == DECAY_SCALAR_INPUT;
  if (a.beta) {
    if (scalar) return launch_pdl(linear_recurrence_kernel<L, NF, false, true>, grid, SCAN_THREADS, 0, stream, a);
    return launch_pdl(linear_recurrence_kernel<L, NF, true, true>, grid, SCAN_THREADS, 0, stream, a);
  }
  if (scalar) return launch_pdl(linear_recurrence_kernel<L, NF, false, false>, grid, SCAN_THREADS, 0, stream, a);
  return launch_pdl(linear_recurrence_kernel<L, NF, true, false>, grid, SCAN_THREADS, 0, stream, a);
}

// z[r][i] = sigmoid(z[r][i] + b[i])^c in place: the decay of gated linear attention from the
// output of its low-rank projection, made once per token and key channel (inside the recurrence
// every block of value channels would make it again).  log sigmoid(x) = -softplus(-x).
__global__ void bias_sigmoid_pow_kernel(float* __restrict__ z, const float* __restrict__ b, long long total,
                                        int n, float c) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float x = z[i] + (b ? b[i % n] : 0.f);
    z[i] = expf(-c * softplus_f(-x));
  }
}

__global__ void rate_decay_kernel(float* __restrict__ z, const float* __restrict__ rate_log,
                                  const float* __restrict__ b, long long total, int n, int per) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % n);
    z[i] = expf(-expf(rate_log[c / per]) * softplus_f(z[i] + (b ? b[c] : 0.f)));
  }
}

// ---- short causal convolution per channel, bias, silu
// out[r][c] = silu(b[c] + sum_{j < taps} w[c][taps - 1 - j] * in(r, j, c)); in(r, j, c) is the input
// of channel c, j tokens before row r: a row of this step when the request has that many rows in
// it before r, else one of the request's last taps - 1 inputs of earlier steps (hist, oldest
// first; zeros at the start of a sequence).
__global__ void causal_conv_silu_kernel(const float* __restrict__ src, int src_stride,
                                        const float* __restrict__ w, const float* __restrict__ b,
                                        const float* __restrict__ hist, long long hist_stride,
                                        const int* __restrict__ row_slot, const int* __restrict__ seg,
                                        int single, float* __restrict__ out, int out_stride, int C, int taps,
                                        int act) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x, r = blockIdx.x;
  if (c >= C) return;
  const int slot = row_slot[r];
  const int before = single ? 0 : r - seg[SEG * slot];       // rows of the request in this step before r
  const float* hrow = hist + (size_t)slot * hist_stride + (size_t)c * (taps - 1);
  float acc = b ? b[c] : 0.f;
  for (int j = taps - 1; j >= 0; --j) {       // oldest input first
    const float x = j <= before ? src[(size_t)(r - j) * src_stride + c] : hrow[taps - 1 - (j - before)];
    acc = fmaf(w[(size_t)c * taps + taps - 1 - j], x, acc);
  }
  out[(size_t)r * out_stride + c] = act ? silu_f(acc) : acc;
}

// The same for 2 to 4 taps with a thread walking a strip of rows of its channel: the weights and
// the last inputs stay in registers, so a row costs one load and one store.  The order of the
// sum is that of the kernel above (oldest input first), so both give the same bits.
template <int TAPS>
__global__ void causal_conv_silu_strip_kernel(const float* __restrict__ src, int src_stride,
                                              const float* __restrict__ w, const float* __restrict__ b,
                                              const float* __restrict__ hist, long long hist_stride,
                                              const int* __restrict__ row_slot, const int* __restrict__ seg,
                                              int single, float* __restrict__ out, int out_stride, int rows,
                                              int C, int act) {
  constexpr int R = 16;
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int r0 = blockIdx.x * R, r1 = min(rows, r0 + R);
  float wt[TAPS], win[TAPS];     // win[j - 1]: the input j rows back, when that row is in the strip
#pragma unroll
  for (int j = 0; j < TAPS; ++j) wt[j] = w[(size_t)c * TAPS + j], win[j] = 0.f;
  const float bias = b ? b[c] : 0.f;
  for (int r = r0; r < r1; ++r) {
    const int slot = row_slot[r];
    const int before = single ? 0 : r - seg[SEG * slot];
    const float x0 = src[(size_t)r * src_stride + c];
    float acc = bias;
#pragma unroll
    for (int j = TAPS - 1; j >= 1; --j) {
      float x;
      if (j <= before) x = r - j >= r0 ? win[j - 1] : src[(size_t)(r - j) * src_stride + c];
      else x = hist[(size_t)slot * hist_stride + (size_t)c * (TAPS - 1) + TAPS - 1 - (j - before)];
      acc = fmaf(wt[TAPS - 1 - j], x, acc);
    }
    acc = fmaf(wt[TAPS - 1], x0, acc);
    out[(size_t)r * out_stride + c] = act ? silu_f(acc) : acc;
#pragma unroll
    for (int j = TAPS - 1; j >= 1; --j) win[j] = win[j - 1];
    win[0] = x0;
  }
}

// hist[slot][c][:] = the last taps - 1 inputs of the request after this step.  A thread owns one
// (request, channel): it reads the old values it still needs before it overwrites them.
__global__ void conv_history_kernel(const float* __restrict__ src, int src_stride, float* __restrict__ hist,
                                    long long hist_stride, const int* __restrict__ row_slot,
                                    const int* __restrict__ seg, int single, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  int slot, first, end;
  if (single) {
    first = blockIdx.x, end = first + 1, slot = row_slot[first];
  } else {
    slot = blockIdx.x;
    first = seg[SEG * slot], end = seg[SEG * slot + 1];
  }
  const int n = end - first;
  if (n <= 0) return;
  float* hrow = hist + (size_t)slot * hist_stride + (size_t)c * (taps - 1);
  for (int i = 0; i < taps - 1; ++i) {      // ascending: hrow[n + i] is read before it is written
    const int at = n + i;                   // index in (old history, then the step's inputs)
    hrow[i] = at < taps - 1 ? hrow[at] : src[(size_t)(first + at - (taps - 1)) * src_stride + c];
  }
}

// ---- gate and group norm behind the recurrence, one block per (row, group of `group` channels)
//   y = o (+ skip[ch / head] * x)                        the recurrence's output, plus a direct path
//   gate_first:  out = unit(y * silu(g)) * w             (the gate comes before the norm)
//   otherwise:   out = unit(y) * w * silu(g)
// (gate_sigmoid: sigmoid(g) in the place of silu(g))
// unit(.) divides a group by its root mean square (eps inside the root); w is indexed by the
// channel modulo w_period (a weight per channel, or one per position in a head shared by heads).
// A thread keeps up to GN_KEEP of its values between the sum and the scaling; a group larger
// than GN_KEEP * THREADS reads the rest twice.
constexpr int GN_KEEP = 8;
__device__ __forceinline__ float gate_f(float z, int sigmoid) {
  const float sg = 1.f / (1.f + expf(-z));
  return sigmoid ? sg : z * sg;
}
template <typename TOut, int THREADS>
__global__ void __launch_bounds__(THREADS) gated_group_norm_kernel(
    const float* __restrict__ o, int o_stride, const float* __restrict__ x, int x_stride,
    const float* __restrict__ skip, int head, const float* __restrict__ g, int g_stride,
    const float* __restrict__ w, int w_period, TOut* __restrict__ out, int out_stride, int groups, int group,
    float eps, int gate_first, int gate_sigmoid) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x / groups, gi = blockIdx.x - r * groups;
  const int c0 = gi * group;
  float y[GN_KEEP], gate[GN_KEEP];
  float ss = 0.f;
  auto value = [&](int ch, float& gt) {
    float v = o[(size_t)r * o_stride + ch];
    if (skip) v = fmaf(skip[ch / head], x[(size_t)r * x_stride + ch], v);
    gt = gate_f(g[(size_t)r * g_stride + ch], gate_sigmoid);
    if (gate_first) v *= gt;
    return v;
  };
#pragma unroll
  for (int n = 0; n < GN_KEEP; ++n) {
    const int i = threadIdx.x + n * THREADS;
    y[n] = 0.f, gate[n] = 0.f;
    if (i < group) {
      y[n] = value(c0 + i, gate[n]);
      ss = fmaf(y[n], y[n], ss);
    }
  }
  for (int i = threadIdx.x + GN_KEEP * THREADS; i < group; i += THREADS) {
    float gt;
    const float v = value(c0 + i, gt);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)group + eps);
#pragma unroll
  for (int n = 0; n < GN_KEEP; ++n) {
    const int i = threadIdx.x + n * THREADS;
    if (i < group) {
      const int ch = c0 + i;
      float v = y[n] * scale * w[ch % w_period];
      if (!gate_first) v *= gate[n];
      out[(size_t)r * out_stride + ch] = from_f32<TOut>(v);
    }
  }
  for (int i = threadIdx.x + GN_KEEP * THREADS; i < group; i += THREADS) {
    const int ch = c0 + i;
    float gt;
    float v = value(ch, gt) * scale * w[ch % w_period];
    if (!gate_first) v *= gt;
    out[(size_t)r * out_stride + ch] = from_f32<TOut>(v);
  }
}
// The same with 16-byte reads: the group, every row stride, the head size and the weight's
// period are multiples of four, so four neighbouring channels share a head and lie together.
template <typename TOut, int THREADS>
__global__ void __launch_bounds__(THREADS) gated_group_norm_vec_kernel(
    const float* __restrict__ o, int o_stride, const float* __restrict__ x, int x_stride,
    const float* __restrict__ skip, int head, const float* __restrict__ g, int g_stride,
    const float* __restrict__ w, int w_period, TOut* __restrict__ out, int out_stride, int groups, int group,
    float eps, int gate_first, int gate_sigmoid) {
  constexpr int KEEP = 2;
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x / groups, gi = blockIdx.x - r * groups;
  const int c0 = gi * group, n4 = group >> 2;
  auto value = [&](int ch, float4& gt) {
    float4 v = *reinterpret_cast<const float4*>(o + (size_t)r * o_stride + ch);
    if (skip) {
      const float d = skip[ch / head];
      const float4 xv = *reinterpret_cast<const float4*>(x + (size_t)r * x_stride + ch);
      v.x = fmaf(d, xv.x, v.x), v.y = fmaf(d, xv.y, v.y), v.z = fmaf(d, xv.z, v.z), v.w = fmaf(d, xv.w, v.w);
    }
    const float4 gv = *reinterpret_cast<const float4*>(g + (size_t)r * g_stride + ch);
    gt = make_float4(gate_f(gv.x, gate_sigmoid), gate_f(gv.y, gate_sigmoid), gate_f(gv.z, gate_sigmoid),
                     gate_f(gv.w, gate_sigmoid));
    if (gate_first) v.x *= gt.x, v.y *= gt.y, v.z *= gt.z, v.w *= gt.w;
    return v;
  };
  auto store = [&](int ch, float4 v, const float4& gt, float scale) {
    const float4 wv = *reinterpret_cast<const float4*>(w + ch % w_period);
    v.x = v.x * scale * wv.x, v.y = v.y * scale * wv.y, v.z = v.z * scale * wv.z, v.w = v.w * scale * wv.w;
    if (!gate_first) v.x *= gt.x, v.y *= gt.y, v.z *= gt.z, v.w *= gt.w;
    TOut* dst = out + (size_t)r * out_stride + ch;
    if (sizeof(TOut) == 4) {
      *reinterpret_cast<float4*>(dst) = v;
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst) = packed;
    }
  };
  float4 y[KEEP], gate[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int n = 0; n < KEEP; ++n) {
    const int i = threadIdx.x + n * THREADS;
    if (i < n4) {
      y[n] = value(c0 + 4 * i, gate[n]);
      ss += y[n].x * y[n].x + y[n].y * y[n].y + y[n].z * y[n].z + y[n].w * y[n].w;
    }
  }
  for (int i = threadIdx.x + KEEP * THREADS; i < n4; i += THREADS) {
    float4 gt;
    const float4 v = value(c0 + 4 * i, gt);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)group + eps);
#pragma unroll
  for (int n = 0; n < KEEP; ++n) {
    const int i = threadIdx.x + n * THREADS;
    if (i < n4) store(c0 + 4 * i, y[n], gate[n], scale);
  }
  for (int i = threadIdx.x + KEEP * THREADS; i < n4; i += THREADS) {
    float4 gt;
    const float4 v = value(c0 + 4 * i, gt);
    store(c0 + 4 * i, v, gt, scale);
  }
}

// ---- exponential gates kept in range by a running maximum (the gates of a matrix memory)
//   i_t = cap tanh((zi_t + bi) / cap),  f_t = log sigmoid(cap tanh((zf_t + bf) / cap))
//   m_t = max(f_t + m_{t-1}, i_t),  keep_t = exp(f_t + m_{t-1} - m_t),  take_t = exp(i_t - m_t)
// per (request, head); m is carried in the request's state slot and starts at 0.  One warp per
// (request of the step, head): the lanes make i and f of 32 tokens at a time, then the chain of
// maxima is walked token by token (every lane walks it; lane j keeps what belongs to token j), so
// the result is that of the token-by-token recurrence however the prompt was cut.
// out[row][0:H] = keep, [H:2H] = take, [2H:3H] = m.
__device__ __forceinline__ float log_sigmoid_f(float z) { return -softplus_f(-z); }
__global__ void __launch_bounds__(32) log_gate_scan_kernel(
    const float* __restrict__ zi, const float* __restrict__ zf, int z_stride, const float* __restrict__ bi,
    const float* __restrict__ bf, float cap, float* __restrict__ m_state, long long state_stride,
    float* __restrict__ out, int out_stride, const int* __restrict__ seg, const int* __restrict__ row_slot,
    int single, int H) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, lane = threadIdx.x;
  int slot, first, end;
  if (single) {
    first = blockIdx.x, end = first + 1, slot = row_slot[first];
  } else {
    slot = seg[SEG * blockIdx.x + 2];
    if (slot < 0) return;
    first = seg[SEG * slot], end = seg[SEG * slot + 1];
  }
  if (end <= first) return;
  float* mp = m_state + (size_t)slot * state_stride + h;
  float m = *mp;
  const float b_i = bi ? bi[h] : 0.f, b_f = bf ? bf[h] : 0.f;
  for (int t0 = first; t0 < end; t0 += 32) {
    const int t = t0 + lane, n = min(32, end - t0);
    float gi = 0.f, gf = 0.f;
    if (t < end) {
      const float a = zi[(size_t)t * z_stride + h] + b_i, b = zf[(size_t)t * z_stride + h] + b_f;
      gi = cap > 0.f ? cap * tanhf(a / cap) : a;
      gf = log_sigmoid_f(cap > 0.f ? cap * tanhf(b / cap) : b);
    }
    float m_before = m, m_mine = m;
    for (int j = 0; j < n; ++j) {
      const float fj = __shfl_sync(0xffffffffu, gf, j), ij = __shfl_sync(0xffffffffu, gi, j);
      const float m_new = fmaxf(fj + m, ij);
      if (j == lane) m_before = m, m_mine = m_new;
      m = m_new;
    }
    if (t < end) {
      float* o = out + (size_t)t * out_stride + h;
      o[0] = expf(gf + m_before - m_mine);
      o[H] = expf(gi - m_mine);
      o[2 * H] = m_mine;
    }
  }
  if (lane == 0) *mp = m;
}

// ---- the output of a matrix memory: normaliser, unit norm per head, gain, sigmoid gate
//   y = o / (max(|z|, exp(-m)) + floor);  out = y / rms(y) * w * sigmoid(g)
// o[row][h][0:V] is the memory's answer and o[row][h][V] = z its normaliser's (both from the
// recurrence above, whose last state column was fed ones); m[row][h] the running maximum of the
// gates.  One warp per (row, head); w has a gain per channel of every head.
template <typename TOut>
__global__ void __launch_bounds__(128) memory_out_norm_kernel(
    const float* __restrict__ o, int o_stride, const float* __restrict__ m, int m_stride,
    const float* __restrict__ g, int g_stride, const float* __restrict__ w, TOut* __restrict__ out,
    int out_stride, long long items, int H, int V, float eps, float floor_) {
  pdl_trigger();
  pdl_wait();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const int r = (int)(item / H), h = (int)(item % H);
  const float* orow = o + (size_t)r * o_stride + (size_t)h * (V + 1);
  const float den = fmaxf(fabsf(orow[V]), expf(-m[(size_t)r * m_stride + h])) + floor_;
  float ss = 0.f;
  for (int j = lane; j < V; j += 32) {
    const float y = orow[j] / den;
    ss = fmaf(y, y, ss);
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)V + eps);
  for (int j = lane; j < V; j += 32) {
    const int ch = h * V + j;
    const float gate = 1.f / (1.f + expf(-g[(size_t)r * g_stride + ch]));
    out[(size_t)r * out_stride + ch] = from_f32<TOut>(orow[j] / den * scale * w[ch] * gate);
  }
}
}  // namespace

LLM_EXPORT int llm_log_gate_scan(const float* zi, const float* zf, int z_stride, const float* bi,
                                 const float* bf, float cap, float* m_state, long long state_stride,
                                 float* out, int out_stride, const int* seg, const int* row_slot, int rows,
                                 int n_requests, int single, int H, cudaStream_t stream) {
  if (rows <= 0 || H <= 0) return 0;
  if (!single && (!seg || n_requests <= 0)) return LLM_ERR_ARGUMENT;
  return launch_pdl(log_gate_scan_kernel, dim3(single ? rows : n_requests, H), 32, 0, stream, zi, zf, z_stride,
                    bi, bf, cap, m_state, state_stride, out, out_stride, seg, row_slot, single, H);
}

LLM_EXPORT int llm_memory_out_norm(const float* o, int o_stride, const float* m, int m_stride, const float* g,
                                   int g_stride, const float* w, void* out, int out_dtype, int out_stride,
                                   int rows, int H, int V, float eps, float floor_, cudaStream_t stream) {
  const long long items = (long long)rows * H;
  if (items <= 0 || V <= 0) return 0;
  const int blocks = (int)((items + 3) / 4);
  if (out_dtype == LLM_F32)
    return launched_many_blocks(launch_pdl(memory_out_norm_kernel<float>, blocks, 128, 0, stream, o, o_stride, m,
                                           m_stride, g, g_stride, w, (float*)out, out_stride, items, H, V, eps,
                                           floor_), blocks);
  if (out_dtype == LLM_BF16)
    return launched_many_blocks(launch_pdl(memory_out_norm_kernel<bf16>, blocks, 128, 0, stream, o, o_stride, m,
                                           m_stride, g, g_stride, w, (bf16*)out, out_stride, items, H, V, eps,
                                           floor_), blocks);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_segment_table(const int* row_slot, int rows, int* seg, int n_slots, cudaStream_t stream) {
  if (n_slots <= 0) return 0;
  return launch_pdl(segment_table_kernel, 1, 256, 0, stream, row_slot, rows, seg, n_slots);
}


// ---- the delta rule over portions of prompts, four tokens at a time.
// With a_m the decay of token m of a group 0..3, A_j = a_0 .. a_j and D_ij = a_(i+1) .. a_j (channel
// by channel), the state S before the group answers token j's key with S^T (A_j k_j) plus, for every
// earlier token i of the group, u_i G_ij with G_ij = sum_e k_i D_ij k_j; its query likewise with
// H_ij = sum_e k_i D_ij q_j (i <= j); and after the group S = A_3 S + sum_i (D_i3 k_i) u_i^T.  So the
// writes u_0 .. u_3 follow from the state's eight answers by a triangular system whose coefficients
// are dot products over the key channels.  Everything a group needs besides the state is made once
// per (request, head, group) by delta_prepare_kernel, in parallel over the tokens: A_j q_j (qa),
// A_j k_j (ka), D_j3 k_j (kh), A_3 (at, for a decay per channel; else the 41st coefficient), the
// coefficients coef[i][0][j] = G_ij (j > i) and coef[i][1][j] = H_ij (j >= i), zero elsewhere, and
// the sigmoid of the write strength (bs); q and k are made unit vectors on the way.  A group's data
// stand at its first row.  delta_groups_kernel then walks the groups of a request in order.
constexpr int GROUP_COEF = 40;      // 32 coefficients, the scalar A_3, padding to whole 16 bytes
constexpr int PREPARE_WARPS = 8, PREPARE_SPLITS = 8;
struct GroupArgs {
  const float* q; int q_stride; const float* k; int k_stride; const float* v; int v_stride;
  const float* d; int d_stride;          // DECAY_VECTOR: the decay [row][h * K + i]; DECAY_RATE_STEP: [row][h]
  const float* beta; int beta_stride;
  const float* p0; const float* p1;
  float q_scale; int unit; float unit_floor;
  const int* seg;
  int H, G, K, V, kind;
  float *qa, *ka, *kh, *at, *coef, *bs;  // [rows][H][K] (four of them), [rows][H][GROUP_COEF], [rows][H]
  float* state; long long state_stride; float* out; int out_stride;
};

__global__ void __launch_bounds__(PREPARE_WARPS * 32) delta_prepare_kernel(const GroupArgs a) {
  pdl_trigger();
  pdl_wait();
  const int slot = a.seg[SEG * blockIdx.x + 2];
  if (slot < 0) return;
  const int first = a.seg[SEG * slot], end = a.seg[SEG * slot + 1];
  const int n_groups = (end - first) >> 2;
  const int h = blockIdx.y, g = h / (a.H / a.G), K = a.K, lane = threadIdx.x & 31;
  const bool vec = a.kind == DECAY_VECTOR;
  const float rate = vec ? 0.f : expf(a.p0[h]), bias = vec ? 0.f : a.p1[h];
  for (int mc = blockIdx.z * PREPARE_WARPS + (threadIdx.x >> 5); mc < n_groups; mc += PREPARE_WARPS * gridDim.z) {
    const int r0 = first + 4 * mc;
    const float *qp[4], *kp[4], *dp[4];
    float as[4] = {1.f, 1.f, 1.f, 1.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      qp[j] = a.q + (size_t)(r0 + j) * a.q_stride + g * K, kp[j] = a.k + (size_t)(r0 + j) * a.k_stride + g * K;
      dp[j] = a.d + (size_t)(r0 + j) * a.d_stride + (vec ? h * K : h);
      if (!vec) as[j] = expf(-rate * softplus_f(dp[j][0] + bias));
    }
    float acc[24];      // 0-3 |q_j|^2, 4-7 |k_j|^2, 8-13 G_ij (i < j), 14-23 H_ij (i <= j), both by rows
#pragma unroll
    for (int x = 0; x < 24; ++x) acc[x] = 0.f;
    for (int i = lane; i < K; i += 32) {
      float qv[4], kv[4], av[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        qv[j] = qp[j][i], kv[j] = kp[j][i], av[j] = vec ? dp[j][i] : as[j];
        acc[j] = fmaf(qv[j], qv[j], acc[j]);
        acc[4 + j] = fmaf(kv[j], kv[j], acc[4 + j]);
      }
      int gi = 8, hi = 14;
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
        float dk = kv[ii];
        acc[hi] = fmaf(dk, qv[ii], acc[hi]), ++hi;
#pragma unroll
        for (int jj = ii + 1; jj < 4; ++jj) {
          dk *= av[jj];
          acc[gi] = fmaf(dk, kv[jj], acc[gi]), ++gi;
          acc[hi] = fmaf(dk, qv[jj], acc[hi]), ++hi;
        }
      }
    }
#pragma unroll
    for (int x = 0; x < 24; ++x) acc[x] = warp_sum(acc[x]);
    float fq[4], fk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      fq[j] = (a.unit ? 1.0f / sqrtf(acc[j] + a.unit_floor) : 1.f) * a.q_scale;
      fk[j] = a.unit ? 1.0f / sqrtf(acc[4 + j] + a.unit_floor) : 1.f;
    }
    if (lane == 0) {
      float* cf = a.coef + ((size_t)r0 * a.H + h) * GROUP_COEF;
      int gi = 8, hi = 14;
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) {
#pragma unroll
        for (int jj = 0; jj < ii; ++jj) cf[ii * 8 + jj] = 0.f, cf[ii * 8 + 4 + jj] = 0.f;
        cf[ii * 8 + ii] = 0.f;
        cf[ii * 8 + 4 + ii] = acc[hi] * fk[ii] * fq[ii], ++hi;
#pragma unroll
        for (int jj = ii + 1; jj < 4; ++jj) {
          cf[ii * 8 + jj] = acc[gi] * fk[ii] * fk[jj], ++gi;
          cf[ii * 8 + 4 + jj] = acc[hi] * fk[ii] * fq[jj], ++hi;
        }
      }
      cf[32] = as[0] * as[1] * as[2] * as[3];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        a.bs[(size_t)(r0 + j) * a.H + h] = 1.f / (1.f + expf(-a.beta[(size_t)(r0 + j) * a.beta_stride + h]));
    }
    for (int i = lane; i < K; i += 32) {
      float qv[4], kv[4], av[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) qv[j] = qp[j][i] * fq[j], kv[j] = kp[j][i] * fk[j], av[j] = vec ? dp[j][i] : as[j];
      float up = 1.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        up *= av[j];
        const size_t at = ((size_t)(r0 + j) * a.H + h) * K + i;
        a.qa[at] = up * qv[j], a.ka[at] = up * kv[j];
      }
      float down = 1.f;
#pragma unroll
      for (int j = 3; j >= 0; --j) {
        a.kh[((size_t)(r0 + j) * a.H + h) * K + i] = down * kv[j];
        down *= av[j];
      }
      if (vec) a.at[((size_t)r0 * a.H + h) * K + i] = up;
    }
  }
}

// A block owns sixteen value channels of one head of one request, as in the kernel above with a
// whole warp per group of four columns.  Per group of four tokens the thirty-two sums (the state's
// answers for four keys and four queries, in four columns) are made in one pass and summed over
// the warp so that lane (kind, token j, column c) = (bit 4, bits 3-2, bits 1-0) ends up with one of
// them; four rounds hand the writes on (the lanes of a key's sum turn it into the write when its
// round comes, the others add what the write does to their sum); then every lane takes all sixteen
// writes and brings its part of the state to the end of the group.  Two groups are staged at a
// time by asynchronous copies, two stages in flight.
template <int NF, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS) delta_groups_kernel(const GroupArgs a) {
  constexpr int L = 32, KP = 4 * L * NF, COLS = 4 * (SCAN_THREADS / 32);
  constexpr int TC = NF == 1 ? 8 : 4, NG = TC / 4;
  __shared__ __align__(16) float qa_s[2][TC][KP];
  __shared__ __align__(16) float ka_s[2][TC][KP];
  __shared__ __align__(16) float kh_s[2][TC][KP];
  __shared__ __align__(16) float at_s[2][VEC ? NG : 1][VEC ? KP : 4];
  __shared__ __align__(16) float coef_s[2][NG][GROUP_COEF];
  __shared__ __align__(16) float v_s[2][TC][COLS];
  __shared__ float b_s[2][TC];
  pdl_trigger();
  pdl_wait();
  const int slot = a.seg[SEG * blockIdx.x + 2];
  if (slot < 0) return;
  const int first = a.seg[SEG * slot];
  const int end = first + ((a.seg[SEG * slot + 1] - first) & ~3);       // whole groups only
  if (end <= first) return;
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = a.K, V = a.V, H = a.H;
  const int j0 = blockIdx.z * COLS, c0 = warp * 4, jc = j0 + c0;
  float* sbase = a.state + (size_t)slot * a.state_stride + (size_t)h * V * K;
  const bool k4 = ((uintptr_t)sbase & 15) == 0;       // (K is a multiple of four here)
  for (int idx = tid; idx < 2 * TC * (KP - K); idx += SCAN_THREADS) {
    const int st = idx / (TC * (KP - K)), rem = idx - st * TC * (KP - K);
    const int tt = rem / (KP - K), i = K + rem - tt * (KP - K);
    qa_s[st][tt][i] = 0.f, ka_s[st][tt][i] = 0.f, kh_s[st][tt][i] = 0.f;
    if (VEC && (tt & 3) == 0) at_s[st][tt >> 2][i] = 1.f;
  }
  auto fetch = [&](int st, int t0) {
    const int n_tok = min(TC, end - t0), k4n = K >> 2;
    for (int idx = tid; idx < n_tok * k4n; idx += SCAN_THREADS) {
      const int tt = idx / k4n, i = (idx - tt * k4n) << 2;
      const size_t at = ((size_t)(t0 + tt) * H + h) * K + i;
      cp_async16(&qa_s[st][tt][i], a.qa + at);
      cp_async16(&ka_s[st][tt][i], a.ka + at);
      cp_async16(&kh_s[st][tt][i], a.kh + at);
      if (VEC && (tt & 3) == 0) cp_async16(&at_s[st][tt >> 2][i], a.at + at);
    }
    for (int idx = tid; idx < (n_tok >> 2) * (GROUP_COEF / 4); idx += SCAN_THREADS) {
      const int gq = idx / (GROUP_COEF / 4), i = (idx - gq * (GROUP_COEF / 4)) << 2;
      cp_async16(&coef_s[st][gq][i], a.coef + ((size_t)(t0 + 4 * gq) * H + h) * GROUP_COEF + i);
    }
    for (int idx = tid; idx < n_tok * COLS; idx += SCAN_THREADS) {
      const int tt = idx / COLS, cc = idx - tt * COLS;
      if (j0 + cc < V) cp_async4(&v_s[st][tt][cc], a.v + (size_t)(t0 + tt) * a.v_stride + h * V + j0 + cc);
      else v_s[st][tt][cc] = 0.f;
    }
    for (int tt = tid; tt < n_tok; tt += SCAN_THREADS) cp_async4(&b_s[st][tt], a.bs + (size_t)(t0 + tt) * H + h);
    cp_async_commit();
  };
  fetch(0, first);
  float s[NF][4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const bool live = jc + c < V;
    const float* srow = sbase + (size_t)(live ? jc + c : 0) * K;
#pragma unroll
    for (int n = 0; n < NF; ++n) {
      const int i0 = 4 * (lane + L * n);
      if (live && k4 && i0 + 3 < K) {
        const float4 t = *reinterpret_cast<const float4*>(srow + i0);
        s[n][0][c] = t.x, s[n][1][c] = t.y, s[n][2][c] = t.z, s[n][3][c] = t.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e][c] = (live && i0 + e < K) ? srow[i0 + e] : 0.f;
      }
    }
  }
  const int kind = lane >> 4, j_mine = (lane >> 2) & 3, c_mine = lane & 3;
  int st = 0;
  for (int t0 = first; t0 < end; t0 += TC, st ^= 1) {
    const int n_groups = min(TC, end - t0) >> 2;
    if (t0 + TC < end) {
      fetch(st ^ 1, t0 + TC);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    for (int mc = 0; mc < n_groups; ++mc) {
      const int tb = 4 * mc;
      float v[32];
#pragma unroll
      for (int x = 0; x < 32; ++x) v[x] = 0.f;
#pragma unroll
      for (int n = 0; n < NF; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 kk = *reinterpret_cast<const float4*>(&ka_s[st][tb + j][4 * (lane + L * n)]);
          const float4 qq = *reinterpret_cast<const float4*>(&qa_s[st][tb + j][4 * (lane + L * n)]);
          const float ke[4] = {kk.x, kk.y, kk.z, kk.w}, qe[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              v[4 * j + c] = fmaf(s[n][e][c], ke[e], v[4 * j + c]);
              v[16 + 4 * j + c] = fmaf(s[n][e][c], qe[e], v[16 + 4 * j + c]);
            }
        }
      }
#pragma unroll
      for (int half = 16; half > 0; half >>= 1) {
        const bool hi = (lane & half) != 0;
#pragma unroll
        for (int x = 0; x < half; ++x) {
          const float send = hi ? v[x] : v[x + half], keep = hi ? v[x + half] : v[x];
          v[x] = keep + __shfl_xor_sync(0xffffffffu, send, half);
        }
      }
      float val = v[0];
      const float v_mine = v_s[st][tb + j_mine][c0 + c_mine], b_mine = b_s[st][tb + j_mine];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float u_cand = b_mine * (v_mine - val);
        const float u_j = __shfl_sync(0xffffffffu, u_cand, (j << 2) | c_mine);
        if (kind == 0 && j_mine == j) val = u_cand;
        val = fmaf(coef_s[st][mc][j * 8 + kind * 4 + j_mine], u_j, val);
      }
      if (kind == 1 && jc + c_mine < V)
        a.out[(size_t)(t0 + tb + j_mine) * a.out_stride + h * V + jc + c_mine] = val;
      float ue[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) ue[j][c] = __shfl_sync(0xffffffffu, val, (j << 2) | c);
      const float at1 = VEC ? 1.f : coef_s[st][mc][32];
#pragma unroll
      for (int n = 0; n < NF; ++n) {
        float4 aa = make_float4(at1, at1, at1, at1);
        if (VEC) aa = *reinterpret_cast<const float4*>(&at_s[st][mc][4 * (lane + L * n)]);
        const float ae[4] = {aa.x, aa.y, aa.z, aa.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
          for (int c = 0; c < 4; ++c) s[n][e][c] *= ae[e];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 kk = *reinterpret_cast<const float4*>(&kh_s[st][tb + j][4 * (lane + L * n)]);
          const float ke[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[n][e][c] = fmaf(ke[e], ue[j][c], s[n][e][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if (jc + c >= V) continue;
    float* srow = sbase + (size_t)(jc + c) * K;
#pragma unroll
    for (int n = 0; n < NF; ++n) {
      const int i0 = 4 * (lane + L * n);
      if (k4 && i0 + 3 < K) {
        *reinterpret_cast<float4*>(srow + i0) = make_float4(s[n][0][c], s[n][1][c], s[n][2][c], s[n][3][c]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (i0 + e < K) srow[i0 + e] = s[n][e][c];
      }
    }
  }
}

template <int NF>
int launch_groups(const GroupArgs& a, int n_requests, cudaStream_t stream) {
  constexpr int COLS = 4 * (SCAN_THREADS / 32);
  const dim3 grid(n_requests, a.H, (a.V + COLS - 1) / COLS);
  if (a.kind == DECAY_VECTOR) return launch_pdl(delta_groups_kernel<NF, true>, grid, SCAN_THREADS, 0, stream, a);
  return launch_pdl(delta_groups_kernel<NF, false>, grid, SCAN_THREADS, 0, stream, a);
}

static int run_scan(ScanArgs& a, int rows, int n_requests, cudaStream_t stream) {
  const int bx = a.single ? rows : n_requests;
  const int K = a.K;
  if (K <= 32) return launch_scan<8, 1>(a, bx, stream);
  if (K <= 64) return launch_scan<16, 1>(a, bx, stream);
  if (K <= 128) return launch_scan<32, 1>(a, bx, stream);
  if (K <= 256) return launch_scan<32, 2>(a, bx, stream);
  return launch_scan<32, 4>(a, bx, stream);
}

// The recurrence over the rows of a step (see the top of this file).  `single`: every row is a
// request of its own; else `seg` is the table of llm_segment_table and `n_requests` the number of
// requests that have rows in the step.  The state of a (slot, head) is V x K floats, the key
// channel fastest.  `ones`: v has V - 1 channels per head and the state's last column is fed the
// constant 1, so that it holds the decayed sum of the keys alone and the last output channel is
// its product with the query (the normaliser of a matrix memory).
LLM_EXPORT int llm_linear_recurrence(const float* q, int q_stride, const float* k, int k_stride, const float* v,
                                     int v_stride, const float* d, int d_stride, const float* d2, int ones,
                                     const float* p0, const float* p1, float c, float q_scale, float* state,
                                     long long state_stride, float* out, int out_stride, const int* seg,
                                     const int* row_slot, int rows, int n_requests, int single, int H, int G,
                                     int K, int V, int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || K <= 0 || V <= 0 || kind < 0 || kind > 3) return LLM_ERR_ARGUMENT;
  if (kind == DECAY_RATE_STEP && (!p0 || !p1)) return LLM_ERR_ARGUMENT;
  if (kind == DECAY_SCALAR_INPUT && !d2) return LLM_ERR_ARGUMENT;
  if (ones && V < 2) return LLM_ERR_ARGUMENT;
  if (!single && (!seg || n_requests <= 0)) return LLM_ERR_ARGUMENT;
  if (K > 512) return LLM_ERR_UNSUPPORTED;     // (sixty-four state registers per lane are the most)
  ScanArgs a;
  a.q = q, a.q_stride = q_stride, a.k = k, a.k_stride = k_stride, a.v = v, a.v_stride = v_stride;
  a.d = d, a.d_stride = d_stride, a.p0 = p0, a.p1 = p1, a.c = c, a.q_scale = q_scale;
  a.d2 = d2, a.ones = ones ? 1 : 0, a.v_cols = ones ? V - 1 : V;
  a.state = state, a.state_stride = state_stride, a.out = out, a.out_stride = out_stride;
  a.seg = seg, a.row_slot = row_slot;
  a.single = single, a.H = H, a.G = G, a.K = K, a.V = V, a.kind = kind;
  a.beta = nullptr, a.beta_stride = 0, a.unit = 0, a.unit_floor = 0.f, a.tail_only = 0;
  const int rc = run_scan(a, rows, n_requests, stream);
  if (!single) next_launch_plain();      // (whatever follows the walk of a portion)
  return rc;
}

// The gated delta rule over the rows of a step, with the state and the segments of the recurrence
// above:  S <- diag(a_t) S;  u = sigmoid(beta_t) (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t.
// kind DECAY_VECTOR: d [rows][H * K] is the decay itself; DECAY_RATE_STEP: d [rows][H] and
// a = exp(-exp(p0[h]) softplus(d + p1[h])) for all key channels of head h.  beta [rows][H] is read
// before its sigmoid.  `unit`: q and k of every head are divided by sqrt(sum of squares + floor)
// first; q is then multiplied by q_scale.
// `work` (work_floats >= rows * H * (4 K + 41) floats, or null): room for what the groups of four
// tokens need; without it every row goes token by token.
LLM_EXPORT int llm_delta_recurrence_grouped(const float* q, int q_stride, const float* k, int k_stride,
                                            const float* v, int v_stride, const float* d, int d_stride,
                                            const float* beta, int beta_stride, const float* p0, const float* p1,
                                            float q_scale, int unit, float unit_floor, float* state,
                                            long long state_stride, float* out, int out_stride, const int* seg,
                                            const int* row_slot, int rows, int n_requests, int single, int H,
                                            int G, int K, int V, int kind, float* work, long long work_floats,
                                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || K <= 0 || V <= 0 || !beta) return LLM_ERR_ARGUMENT;
  if (kind != DECAY_VECTOR && kind != DECAY_RATE_STEP) return LLM_ERR_ARGUMENT;
  if (kind == DECAY_RATE_STEP && (!p0 || !p1)) return LLM_ERR_ARGUMENT;
  if (!single && (!seg || n_requests <= 0)) return LLM_ERR_ARGUMENT;
  if (K > 512) return LLM_ERR_UNSUPPORTED;
  ScanArgs a;
  a.q = q, a.q_stride = q_stride, a.k = k, a.k_stride = k_stride, a.v = v, a.v_stride = v_stride;
  a.d = d, a.d_stride = d_stride, a.p0 = p0, a.p1 = p1, a.c = 1.f, a.q_scale = q_scale;
  a.d2 = nullptr, a.ones = 0, a.v_cols = V;
  a.state = state, a.state_stride = state_stride, a.out = out, a.out_stride = out_stride;
  a.seg = seg, a.row_slot = row_slot;
  a.single = single, a.H = H, a.G = G, a.K = K, a.V = V, a.kind = kind;
  a.beta = beta, a.beta_stride = beta_stride, a.unit = unit ? 1 : 0, a.unit_floor = unit_floor, a.tail_only = 0;
  // Portions of prompts with 68 to 256 key channels go four tokens at a time: what a group needs
  // is prepared once per head in parallel over the tokens, the walk takes a group per round, and
  // the token-by-token kernel takes the rows that are left (fewer than four a request).
  const long long need = (long long)rows * H * (4LL * K + GROUP_COEF + 1);
  if (!single && work && work_floats >= need && K > 64 && K <= 256 && (K & 3) == 0) {
    GroupArgs ga;
    ga.q = q, ga.q_stride = q_stride, ga.k = k, ga.k_stride = k_stride, ga.v = v, ga.v_stride = v_stride;
    ga.d = d, ga.d_stride = d_stride, ga.beta = beta, ga.beta_stride = beta_stride, ga.p0 = p0, ga.p1 = p1;
    ga.q_scale = q_scale, ga.unit = unit ? 1 : 0, ga.unit_floor = unit_floor, ga.seg = seg;
    ga.H = H, ga.G = G, ga.K = K, ga.V = V, ga.kind = kind;
    const size_t plane = (size_t)rows * H * K;
    ga.qa = work, ga.ka = work + plane, ga.kh = work + 2 * plane, ga.at = work + 3 * plane;
    ga.coef = work + 4 * plane, ga.bs = ga.coef + (size_t)rows * H * GROUP_COEF;
    ga.state = state, ga.state_stride = state_stride, ga.out = out, ga.out_stride = out_stride;
    int rc = launch_pdl(delta_prepare_kernel, dim3(n_requests, H, PREPARE_SPLITS), PREPARE_WARPS * 32, 0, stream, ga);
    if (rc != 0) return rc;
    next_launch_plain();
    rc = K <= 128 ? launch_groups<1>(ga, n_requests, stream) : launch_groups<2>(ga, n_requests, stream);
    if (rc != 0) return rc;
    a.tail_only = 1;
    next_launch_plain();
  }
  const int rc = run_scan(a, rows, n_requests, stream);
  if (!single) next_launch_plain();      // (whatever follows the walk of a portion)
  return rc;
}

// (the form without room for the groups' preparation: token by token throughout)
LLM_EXPORT int llm_delta_recurrence(const float* q, int q_stride, const float* k, int k_stride, const float* v,
                                    int v_stride, const float* d, int d_stride, const float* beta,
                                    int beta_stride, const float* p0, const float* p1, float q_scale, int unit,
                                    float unit_floor, float* state, long long state_stride, float* out,
                                    int out_stride, const int* seg, const int* row_slot, int rows,
                                    int n_requests, int single, int H, int G, int K, int V, int kind,
                                    cudaStream_t stream) {
  return llm_delta_recurrence_grouped(q, q_stride, k, k_stride, v, v_stride, d, d_stride, beta, beta_stride, p0, p1,
                                      q_scale, unit, unit_floor, state, state_stride, out, out_stride, seg,
                                      row_slot, rows, n_requests, single, H, G, K, V, kind, nullptr, 0, stream);
}

// z[r][c] = exp(-exp(rate_log[c / per]) * softplus(z[r][c] + bias[c])) in place: a decay per
// (token, head, key channel) from a projected step size, made once per token (`per` channels
// share a rate).
LLM_EXPORT int llm_rate_decay(float* z, const float* rate_log, const float* bias, int rows, int n, int per,
                              cudaStream_t stream) {
  const long long total = (long long)rows * n;
  if (total <= 0) return 0;
  if (per <= 0 || !rate_log) return LLM_ERR_ARGUMENT;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  return launch_pdl(rate_decay_kernel, blocks, 256, 0, stream, z, rate_log, bias, total, n, per);
}

LLM_EXPORT int llm_bias_sigmoid_pow(float* z, const float* b, int rows, int n, float c, cudaStream_t stream) {
  const long long total = (long long)rows * n;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  return launch_pdl(bias_sigmoid_pow_kernel, blocks, 256, 0, stream, z, b, total, n, c);
}

// The convolution of `C` channels over the rows of a step, then the request's history of inputs
// brought up to date (two launches: the second overwrites what the first reads).
// (act 1: silu behind the sum, 0: the sum as it is)
LLM_EXPORT int llm_causal_conv(const float* src, int src_stride, const float* w, const float* b,
                               float* hist, long long hist_stride, const int* row_slot, const int* seg,
                               int rows, int n_slots, int single, float* out, int out_stride, int C,
                               int taps, int act, cudaStream_t stream) {
  if (rows <= 0 || C <= 0) return 0;
  if (taps < 1 || (!single && !seg)) return LLM_ERR_ARGUMENT;
  int rc;
  const dim3 strips((rows + 15) / 16, (C + 127) / 128);
#define STRIP(T)                                                                                             \
  rc = launch_pdl(causal_conv_silu_strip_kernel<T>, strips, 128, 0, stream, src, src_stride, w, b,            \
                  (const float*)hist, hist_stride, row_slot, seg, single, out, out_stride, rows, C, act)
  // (strips pay from a few hundred rows on; a decode step has too few rows to fill the GPU with them)
  if (taps == 2 && rows >= 256) STRIP(2);
  else if (taps == 3 && rows >= 256) STRIP(3);
  else if (taps == 4 && rows >= 256) STRIP(4);
  else
    rc = launch_pdl(causal_conv_silu_kernel, dim3(rows, (C + 127) / 128), 128, 0, stream, src, src_stride, w, b,
                    (const float*)hist, hist_stride, row_slot, seg, single, out, out_stride, C, taps, act);
#undef STRIP
  if (rc != 0 || taps == 1) return rc;
  return launch_pdl(conv_history_kernel, dim3(single ? rows : n_slots, (C + 127) / 128), 128, 0, stream, src,
                    src_stride, hist, hist_stride, row_slot, seg, single, C, taps);
}

LLM_EXPORT int llm_causal_conv_silu(const float* src, int src_stride, const float* w, const float* b,
                                    float* hist, long long hist_stride, const int* row_slot, const int* seg,
                                    int rows, int n_slots, int single, float* out, int out_stride, int C,
                                    int taps, cudaStream_t stream) {
  return llm_causal_conv(src, src_stride, w, b, hist, hist_stride, row_slot, seg, rows, n_slots, single, out,
                         out_stride, C, taps, 1, stream);
}

// ---- minGRU: a gated recurrence per channel whose gates read only the current token
//   z = sigmoid(zr + bz), u = ur + bx, candidate c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0)
//   S <- (1 - z) S + z c;  out = S * silu(g)                              (all 32-bit)
// The state is carried through memory unrounded.  A step of single tokens takes a thread per
// (row, channel): the gates, one multiply-add, the output.
__device__ __forceinline__ void min_gru_gate(float zr, float ur, float bz, float bx, float& keep, float& add) {
  const float zz = 1.f / (1.f + expf(-(zr + bz)));
  const float uu = ur + bx;
  const float cand = uu >= 0.f ? uu + 0.5f : 1.f / (1.f + expf(-uu));
  keep = 1.f - zz;
  add = zz * cand;
}

template <typename TOut>
__global__ void __launch_bounds__(128) min_gru_token_kernel(
    const float* __restrict__ z, const float* __restrict__ u, const float* __restrict__ g, int stride,
    const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state, long long state_stride,
    TOut* __restrict__ out, int out_stride, const int* __restrict__ row_slot, int width) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x, r = blockIdx.x;
  if (c >= width) return;
  const size_t at = (size_t)r * stride + c;
  float k, a;
  min_gru_gate(z[at], u[at], bz ? bz[c] : 0.f, bx ? bx[c] : 0.f, k, a);
  float* sp = state + (size_t)row_slot[r] * state_stride + c;
  const float S = fmaf(k, *sp, a);
  *sp = S;
  out[(size_t)r * out_stride + c] = from_f32<TOut>(S * silu_f(g[at]));
}

// The same walk for steps that hold portions of prompts: a block per (request, 32 channels) cuts
// the request's rows into as many runs as it has warps.  S <- k S + a is a chain of affine maps, so
// every warp first folds its run into one map (the product of the k and the run's result from
// zero), the maps of the runs before a warp give the state that enters its run, and a second walk
// writes the rows.  The chain a row waits for is 2 / warps of the portion; the sums are 32-bit and
// differ from the token-by-token walk by rounding only.  Rows are taken eight at a time, so that
// their loads and their gates (which do not wait for the chain) overlap.
constexpr int GRU_WARPS = 32;
constexpr int GRU_BATCH = 8;      // rows whose loads and gates are under way together

// It makes the gates in both walks, with the expressions of the kernel above.

template <typename TOut>
__global__ void __launch_bounds__(GRU_WARPS * 32) min_gru_runs_kernel(
    const float* __restrict__ z, const float* __restrict__ u, const float* __restrict__ g, int stride,
    const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state, long long state_stride,
    TOut* __restrict__ out, int out_stride, const int* __restrict__ seg, int width) {
  __shared__ float map_k[GRU_WARPS][32], map_a[GRU_WARPS][32];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.y * 32 + lane, slot = blockIdx.x;
  const int first = seg[SEG * slot], end = seg[SEG * slot + 1];
  if (end <= first) return;
  const bool live = c < width;
  const int n = end - first, per = (n + GRU_WARPS - 1) / GRU_WARPS;
  const int r0 = first + (w * per < n ? w * per : n), r1 = first + ((w + 1) * per < n ? (w + 1) * per : n);
  const float bzc = live && bz ? bz[c] : 0.f, bxc = live && bx ? bx[c] : 0.f;
  float K = 1.f, A = 0.f;
  if (live) {
    for (int r = r0; r < r1; r += GRU_BATCH) {
      float zr[GRU_BATCH], ur[GRU_BATCH];
#pragma unroll
      for (int i = 0; i < GRU_BATCH; ++i) {
        const size_t at = (size_t)(r + i < r1 ? r + i : r1 - 1) * stride + c;
        zr[i] = z[at], ur[i] = u[at];
      }
#pragma unroll
      for (int i = 0; i < GRU_BATCH; ++i) {
        float k, a;
        min_gru_gate(zr[i], ur[i], bzc, bxc, k, a);
        if (r + i < r1) K *= k, A = fmaf(k, A, a);
      }
    }
  }
  map_k[w][lane] = K, map_a[w][lane] = A;
  // (the old state is read on this side of the barrier, the new one written on the other)
  float* sp = state + (size_t)slot * state_stride + (live ? c : 0);
  float S = *sp;
  __syncthreads();
  if (!live) return;
  for (int j = 0; j < w; ++j) S = fmaf(map_k[j][lane], S, map_a[j][lane]);
  for (int r = r0; r < r1; r += GRU_BATCH) {
    float zr[GRU_BATCH], ur[GRU_BATCH], gr[GRU_BATCH];
#pragma unroll
    for (int i = 0; i < GRU_BATCH; ++i) {
      const size_t at = (size_t)(r + i < r1 ? r + i : r1 - 1) * stride + c;
      zr[i] = z[at], ur[i] = u[at], gr[i] = g[at];
    }
#pragma unroll
    for (int i = 0; i < GRU_BATCH; ++i) {
      float k, a;
      min_gru_gate(zr[i], ur[i], bzc, bxc, k, a);
      const float gate = silu_f(gr[i]);
      if (r + i < r1) {
        S = fmaf(k, S, a);
        out[(size_t)(r + i) * out_stride + c] = from_f32<TOut>(S * gate);
      }
    }
  }
  if (w == GRU_WARPS - 1) *sp = S;
}

// z, u, g: three column ranges of one float32 matrix of row stride `stride`;
// state float32 [slots][>= width]; out [rows][width] in out_dtype.
LLM_EXPORT int llm_min_gru(float* z, float* u, float* g, int stride, const float* bz, const float* bx,
                           float* state, long long state_stride, void* out, int out_dtype, int out_stride,
                           const int* row_slot, const int* seg, int rows, int n_slots, int single, int width,
                           cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (!single && !seg) return LLM_ERR_ARGUMENT;
  if (!single) {
    const dim3 grid(n_slots, (width + 31) / 32);
    if (out_dtype == LLM_F32)
      return launch_pdl(min_gru_runs_kernel<float>, grid, GRU_WARPS * 32, 0, stream, (const float*)z,
                        (const float*)u, (const float*)g, stride, bz, bx, state, state_stride, (float*)out,
                        out_stride, seg, width);
    if (out_dtype == LLM_BF16)
      return launch_pdl(min_gru_runs_kernel<bf16>, grid, GRU_WARPS * 32, 0, stream, (const float*)z,
                        (const float*)u, (const float*)g, stride, bz, bx, state, state_stride, (bf16*)out,
                        out_stride, seg, width);
    return LLM_ERR_UNSUPPORTED;
  }
  const dim3 grid(rows, (width + 127) / 128);
  if (out_dtype == LLM_F32)
    return launch_pdl(min_gru_token_kernel<float>, grid, 128, 0, stream, (const float*)z, (const float*)u,
                      (const float*)g, stride, bz, bx, state, state_stride, (float*)out, out_stride, row_slot,
                      width);
  if (out_dtype == LLM_BF16)
    return launch_pdl(min_gru_token_kernel<bf16>, grid, 128, 0, stream, (const float*)z, (const float*)u,
                      (const float*)g, stride, bz, bx, state, state_stride, (bf16*)out, out_stride, row_slot,
                      width);
  return LLM_ERR_UNSUPPORTED;
}

static int gated_group_norm_launch(const float* o, int o_stride, const float* x, int x_stride,
                                   const float* skip, int head, const float* g, int g_stride, const float* w,
                                   int w_period, void* out, int out_dtype, int out_stride, int rows,
                                   int groups, int group, float eps, int gate_first, int gate_sigmoid,
                                   cudaStream_t stream) {
  if (rows <= 0 || groups <= 0) return 0;
  if (group <= 0 || w_period <= 0 || (skip && (!x || head <= 0))) return LLM_ERR_ARGUMENT;
  const long long items = (long long)rows * groups;
  if (items > 0x7fffffffLL) return LLM_ERR_UNSUPPORTED;
  const int blocks = (int)items;
  const bool vec = !((group | o_stride | g_stride | out_stride | w_period) & 3) &&
                   (!skip || !((head | x_stride) & 3)) &&
                   !(((uintptr_t)o | (uintptr_t)g | (uintptr_t)w | (uintptr_t)out | (uintptr_t)x) & 15);
#define GNV(T, TH)                                                                                             \
  return launch_pdl(gated_group_norm_vec_kernel<T, TH>, blocks, TH, 0, stream, o, o_stride, x, x_stride, skip,  \
                    head, g, g_stride, w, w_period, (T*)out, out_stride, groups, group, eps, gate_first,   \
                    gate_sigmoid)
  if (vec && out_dtype == LLM_F32) {
    if (group <= 256) GNV(float, 32);
    if (group <= 512) GNV(float, 64);
    if (group <= 2048) GNV(float, 256);
    GNV(float, 1024);
  }
  if (vec && out_dtype == LLM_BF16) {
    if (group <= 256) GNV(bf16, 32);
    if (group <= 512) GNV(bf16, 64);
    if (group <= 2048) GNV(bf16, 256);
    GNV(bf16, 1024);
  }
#undef GNV
#define GN(T, TH)                                                                                          \
  return launch_pdl(gated_group_norm_kernel<T, TH>, blocks, TH, 0, stream, o, o_stride, x, x_stride, skip,  \
                    head, g, g_stride, w, w_period, (T*)out, out_stride, groups, group, eps, gate_first,   \
                    gate_sigmoid)
  if (out_dtype == LLM_F32) {
    if (group <= 64) GN(float, 32);
    if (group <= 512) GN(float, 64);
    if (group <= 2048) GN(float, 256);
    GN(float, 1024);
  }
  if (out_dtype == LLM_BF16) {
    if (group <= 64) GN(bf16, 32);
    if (group <= 512) GN(bf16, 64);
    if (group <= 2048) GN(bf16, 256);
    GN(bf16, 1024);
  }
#undef GN
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_gated_group_norm_act(const float* o, int o_stride, const float* x, int x_stride,
                                        const float* skip, int head, const float* g, int g_stride, const float* w,
                                        int w_period, void* out, int out_dtype, int out_stride, int rows,
                                        int groups, int group, float eps, int gate_first, int gate_sigmoid,
                                        cudaStream_t stream);

LLM_EXPORT int llm_gated_group_norm(const float* o, int o_stride, const float* x, int x_stride,
                                    const float* skip, int head, const float* g, int g_stride, const float* w,
                                    int w_period, void* out, int out_dtype, int out_stride, int rows,
                                    int groups, int group, float eps, int gate_first, cudaStream_t stream) {
  return llm_gated_group_norm_act(o, o_stride, x, x_stride, skip, head, g, g_stride, w, w_period, out, out_dtype,
                                  out_stride, rows, groups, group, eps, gate_first, 0, stream);
}

// (a kernel of many blocks that stands in front of the output projection: see launched_many_blocks)
LLM_EXPORT int llm_gated_group_norm_act(const float* o, int o_stride, const float* x, int x_stride,
                                        const float* skip, int head, const float* g, int g_stride, const float* w,
                                        int w_period, void* out, int out_dtype, int out_stride, int rows,
                                        int groups, int group, float eps, int gate_first, int gate_sigmoid,
                                        cudaStream_t stream) {
  const int rc = gated_group_norm_launch(o, o_stride, x, x_stride, skip, head, g, g_stride, w, w_period, out,
                                         out_dtype, out_stride, rows, groups, group, eps, gate_first, gate_sigmoid,
                                         stream);
  return launched_many_blocks(rc, (long long)rows * groups);
}

// Persistent LSTM recurrence kernels for sm_100a.
//
// Reference behaviour: the `RNN` operator in lstm mode (src/operator/rnn-inl.h, cudnnRNNForwardTraining /
// cudnnRNNBackwardData / cudnnRNNBackwardWeights; CPU math in src/operator/rnn_impl.h).  Gate order i, f, g, o.
//
// The input projection x_t·W_ihᵀ + b_ih + b_hh of all time steps is one large GEMM done before these kernels
// (tensor cores); what remains is the strictly sequential part
//     a_t = xproj_t + h_{t-1}·W_hhᵀ,  i,f,o = sigmoid(a), g = tanh(a),  c_t = f·c_{t-1} + i·g,  h_t = o·tanh(c_t)
// which is latency-bound: a (batch x H) by (H x 4H) product per step.  One cooperative launch covers all time steps:
//   * every CTA owns a slice of `U` hidden units and keeps the 4U rows of W_hh that produce their gates in shared
//     memory for the whole sequence (no weight traffic per step);
//   * h_{t-1} lives in a k-major exchange buffer in global memory ([H][batch]); per step a CTA streams it through shared
//     memory in tiles with double-buffered 16-byte cp.async copies, each thread owns a pair of batch rows and a residue
//     class of the tile's k rows and multiplies against the resident weights (broadcast reads), partial sums are
//     combined through shared memory, then the cell update of the CTA's units is done in place;
//   * the new h slice goes to the other half of the exchange buffer and all CTAs meet at a grid barrier (an arrival
//     counter with a bounded spin); c and the carried gradients never leave the CTA.
// The backward kernel walks the time steps in reverse with the same ownership: phase A turns dh_t, dc_t into the gate
// gradients of the CTA's units, the barrier publishes them, phase B contracts all 4H gate gradients with the CTA's
// columns of W_hh (also resident in shared memory) to obtain dh_{t-1} for its units.  Weight and input gradients are
// large GEMMs over the saved gate gradients, done outside.
// A barrier that does not complete within its time budget sets an error flag and every CTA leaves the loop.
#include <cooperative_groups.h>

#include "common.cuh"

namespace mxb {

constexpr int kLstmThreads = 256;
constexpr unsigned long long kLstmBarrierNs = 2000000000ull;    // 2 s per barrier

struct LstmParams {
  const void* xproj;     // [T, B, 4H]  x·W_ihᵀ + b_ih + b_hh
  const void* whh;       // [4H, H]
  const void* h0;        // [B, H]
  const void* c0;        // [B, H]
  void* y;               // [T, B, H]
  void* hT;              // [B, H]
  void* cT;              // [B, H]
  void* gates;           // [T, 4H, Bp] activated gates, k-major like the exchange buffer (saved for backward; may be null)
  float* cs;             // [T, H, Bp] cell states in fp32, k-major (saved for backward; may be null)
  void* hbuf;            // forward exchange buffer, k-major: [2][H][Bp] of h
  int Bp;                // batch rounded up to a multiple of 8 (row length of the exchange buffer)
  int tileK;             // rows of the exchange buffer staged in shared memory per copy (two buffers)
  unsigned int* bar;     // [2] arrival counter, error flag
  int T, B, H, U;        // U: hidden units per CTA
  // backward only
  const void* dy;        // [T, B, H]
  const void* dhT;       // [B, H] or null
  const void* dcT;       // [B, H] or null
  void* dgates;          // [T, 4H, Bp] gradient w.r.t. the pre-activation gates, k-major: step t is also the
                         // operand that phase B of that step streams (no separate exchange copy)
  void* dh0;             // [B, H]
  void* dc0;             // [B, H]
  // GRU / vanilla RNN kernels only
  const void* bhn;       // [H] hidden-side bias of the GRU candidate gate (inside r * (...))
  void* hnb;             // [T, H, Bp] h_{t-1}.W_hn + b_hn, k-major (GRU, saved for backward; may be null)
  void* dan;             // [T, H, Bp] gradient w.r.t. the candidate pre-activation, k-major (GRU backward)
  int relu;              // vanilla RNN: 1 = relu, 0 = tanh
};

__device__ __forceinline__ unsigned long long lstm_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// All CTAs arrive; returns false when the others did not show up in time (or an error was already flagged).
__device__ bool grid_barrier(unsigned int* bar, unsigned int target) {
  __shared__ int ok;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    ok = 1;
    atomicAdd(bar, 1u);
    const unsigned long long t0 = lstm_now_ns();
    unsigned spins = 0;
    while ((int)(*(volatile unsigned int*)bar - target) < 0) {
      if (*(volatile unsigned int*)(bar + 1) != 0u) { ok = 0; break; }
      if ((++spins & 63u) == 0 && lstm_now_ns() - t0 > kLstmBarrierNs) {
        atomicExch(bar + 1, 1u);
        ok = 0;
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
  return ok != 0;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ float ldf(const void* p, int64_t i) { return Cvt<T>::to_f(static_cast<const T*>(p)[i]); }
template <typename T>
__device__ __forceinline__ void stf(void* p, int64_t i, float v) { static_cast<T*>(p)[i] = Cvt<T>::from_f(v); }

// ---- streaming a [K][Bp] matrix from global memory through shared memory against resident weights ------------------
// The exchanged operand (h_{t-1}, or the gate gradients of step t) is kept K-major in global memory: row k holds the
// values of all batch rows.  A CTA copies it in tiles of `tileK` rows (as many as the shared memory left over by the
// weights allows, so that few round trips to L2 are exposed) with 16-byte cp.async, double buffered, and every
// thread owns one pair of batch rows and a residue class of the tile's k rows, so a warp reads consecutive words of
// the staged tile (no bank conflicts) and the weight row of that k as a broadcast.
constexpr int kMinTileK = 48;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename X>
__device__ __forceinline__ void issue_tile(const X* __restrict__ src, X* __restrict__ stage, int k0, int K, int Bp, int tileK) {
  const int rows = min(tileK, K - k0);
  const int chunks_per_row = Bp * (int)sizeof(X) / 16;
  const int total = rows * chunks_per_row;
  const char* g = reinterpret_cast<const char*>(src + (int64_t)k0 * Bp);
  char* s = reinterpret_cast<char*>(stage);
  for (int c = threadIdx.x; c < total; c += blockDim.x) cp_async16(s + (size_t)c * 16, g + (size_t)c * 16);
}

// acc[2][OUT] += sum_k src[k][b0 + {0,1}] * W[k][0..OUT) over all K rows; W: shared memory, row stride OUT floats.
template <typename X, int OUT>
__device__ __forceinline__ void stream_matmul(const X* __restrict__ src, int K, int Bp, const float* __restrict__ W,
                                              X* __restrict__ stage /* 2 tiles of tileK*Bp */, int tileK, int kg, int KG,
                                              int b0, bool active, float (&acc)[2][OUT]) {
#pragma unroll
  for (int o = 0; o < OUT; ++o) { acc[0][o] = 0.f; acc[1][o] = 0.f; }
  const int ntiles = (K + tileK - 1) / tileK;
  issue_tile(src, stage, 0, K, Bp, tileK);
  cp_async_commit();
  for (int tile = 0; tile < ntiles; ++tile) {
    X* cur = stage + (size_t)(tile & 1) * tileK * Bp;
    if (tile + 1 < ntiles) {
      issue_tile(src, stage + (size_t)((tile + 1) & 1) * tileK * Bp, (tile + 1) * tileK, K, Bp, tileK);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (active) {
      const int k0 = tile * tileK, rows = min(tileK, K - k0);
      for (int k = kg; k < rows; k += KG) {
        const float x0 = Cvt<X>::to_f(cur[(size_t)k * Bp + b0]), x1 = Cvt<X>::to_f(cur[(size_t)k * Bp + b0 + 1]);
        const float* w = W + (size_t)(k0 + k) * OUT;
        if constexpr (OUT % 4 == 0) {
          const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
          for (int q = 0; q < OUT / 4; ++q) {
            const float4 wv = w4[q];
            acc[0][4 * q] += x0 * wv.x; acc[0][4 * q + 1] += x0 * wv.y; acc[0][4 * q + 2] += x0 * wv.z; acc[0][4 * q + 3] += x0 * wv.w;
            acc[1][4 * q] += x1 * wv.x; acc[1][4 * q + 1] += x1 * wv.y; acc[1][4 * q + 2] += x1 * wv.z; acc[1][4 * q + 3] += x1 * wv.w;
          }
        } else {
#pragma unroll
          for (int o = 0; o < OUT; ++o) {
            const float wv = w[o];
            acc[0][o] += x0 * wv;
            acc[1][o] += x1 * wv;
          }
        }
      }
    }
    __syncthreads();          // the tile may be overwritten by the copy issued in the next trip
  }
}

// Forward.  Shared memory: Wt [H][4U] (W_hh rows of this CTA's units, k-major), red [KG][Bp][4U], cst [Bp][U],
// stage [2][tileK][Bp] of the exchange type X (float for fp32 models, T otherwise).
template <typename T, typename X, int U>
__global__ void __launch_bounds__(kLstmThreads) lstm_fwd_kernel(const LstmParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, B = p.B, Bp = p.Bp;
  constexpr int R = 4 * U;
  const int j0 = blockIdx.x * U;
  const int nu = min(U, H - j0);
  const int NB2 = Bp / 2;
  const int KG = max(1, kLstmThreads / NB2);
  float* Wt = reinterpret_cast<float*>(smem_raw);                 // [H][R]
  float* red = Wt + (size_t)H * R;                                // [KG][Bp][R]
  float* cst = red + (size_t)KG * Bp * R;                         // [Bp][U]
  X* stage = reinterpret_cast<X*>(cst + (size_t)Bp * U);          // [2][tileK][Bp]
  X* hx = static_cast<X*>(p.hbuf);                                // [2][H][Bp] k-major exchange buffer
  for (int idx = threadIdx.x; idx < H * R; idx += blockDim.x) {
    const int k = idx / R, r = idx % R;
    const int g = r / U, jj = r % U;
    Wt[idx] = jj < nu ? ldf<T>(p.whh, (int64_t)(g * H + j0 + jj) * H + k) : 0.f;
  }
  for (int idx = threadIdx.x; idx < Bp * U; idx += blockDim.x) {
    const int b = idx / U, jj = idx % U;
    cst[idx] = (jj < nu && b < B) ? ldf<T>(p.c0, (int64_t)b * H + j0 + jj) : 0.f;
  }
  for (int idx = threadIdx.x; idx < Bp * nu; idx += blockDim.x) {    // h_{-1} into slot 0 (padding rows = 0)
    const int jj = idx / Bp, b = idx % Bp;
    hx[(int64_t)(j0 + jj) * Bp + b] = Cvt<X>::from_f(b < B ? ldf<T>(p.h0, (int64_t)b * H + j0 + jj) : 0.f);
  }
  unsigned int target = gridDim.x;
  bool alive = grid_barrier(p.bar, target);
  const int kg = threadIdx.x / NB2, b0 = (threadIdx.x % NB2) * 2;
  const bool active = kg < KG;
  for (int t = 0; t < p.T && alive; ++t) {
    const X* hprev = hx + (int64_t)(t & 1) * H * Bp;
    X* hnext = hx + (int64_t)((t + 1) & 1) * H * Bp;
    // this step's input projections for the (at most two) cells this thread will update: issued before the product
    // so that their latency is hidden behind it
    float xp[2][4];
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int idx = threadIdx.x + it * kLstmThreads;
      const int jj = idx / Bp, b = idx % Bp;
#pragma unroll
      for (int g = 0; g < 4; ++g)
        xp[it][g] = (idx < Bp * nu && b < B) ? ldf<T>(p.xproj, ((int64_t)t * B + b) * 4 * H + g * H + j0 + jj) : 0.f;
    }
    float acc[2][R];
    stream_matmul<X, R>(hprev, H, Bp, Wt, stage, p.tileK, kg, KG, b0, active, acc);
    if (active) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float* dst = red + ((size_t)kg * Bp + b0 + rr) * R;
#pragma unroll
        for (int o = 0; o < R; ++o) dst[o] = acc[rr][o];
      }
    }
    __syncthreads();
    auto update_cell = [&](int idx, const float (&xg)[4]) {
      const int jj = idx / Bp, b = idx % Bp, j = j0 + jj;
      if (b >= B) { hnext[(int64_t)j * Bp + b] = Cvt<X>::from_f(0.f); return; }
      float a[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float s = xg[g];
        for (int q = 0; q < KG; ++q) s += red[((size_t)q * Bp + b) * R + g * U + jj];
        a[g] = s;
      }
      const float ig = sigmoidf_(a[0]), fg = sigmoidf_(a[1]), gg = tanhf(a[2]), og = sigmoidf_(a[3]);
      const float c = fg * cst[b * U + jj] + ig * gg;
      const float h = og * tanhf(c);
      cst[b * U + jj] = c;
      hnext[(int64_t)j * Bp + b] = Cvt<X>::from_f(h);
      stf<T>(p.y, ((int64_t)t * B + b) * H + j, h);
      if (p.gates) {        // consecutive threads = consecutive batch rows: contiguous stores
        const int64_t gb = ((int64_t)t * 4 * H + j) * Bp + b, gs = (int64_t)H * Bp;
        stf<T>(p.gates, gb, ig); stf<T>(p.gates, gb + gs, fg); stf<T>(p.gates, gb + 2 * gs, gg); stf<T>(p.gates, gb + 3 * gs, og);
      }
      if (p.cs) p.cs[((int64_t)t * H + j) * Bp + b] = c;
      if (t == p.T - 1) { stf<T>(p.hT, (int64_t)b * H + j, h); stf<T>(p.cT, (int64_t)b * H + j, c); }
    };
    if ((int)threadIdx.x < Bp * nu) update_cell(threadIdx.x, xp[0]);
    if ((int)threadIdx.x + kLstmThreads < Bp * nu) update_cell(threadIdx.x + kLstmThreads, xp[1]);
    for (int idx = threadIdx.x + 2 * kLstmThreads; idx < Bp * nu; idx += blockDim.x) {
      const int jj = idx / Bp, b = idx % Bp;
      float xg[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) xg[g] = b < B ? ldf<T>(p.xproj, ((int64_t)t * B + b) * 4 * H + g * H + j0 + jj) : 0.f;
      update_cell(idx, xg);
    }
    target += gridDim.x;
    alive = grid_barrier(p.bar, target);
  }
}

// Backward.  Shared memory: Wc [4H][U] (columns of W_hh of this CTA's units), red [KG][Bp][U], dh_rec [Bp][U],
// dc_car [Bp][U], stage [2][tileK][Bp].
template <typename T, typename X, int U>
__global__ void __launch_bounds__(kLstmThreads) lstm_bwd_kernel(const LstmParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, B = p.B, Bp = p.Bp, H4 = 4 * p.H;
  const int j0 = blockIdx.x * U;
  const int nu = min(U, H - j0);
  const int NB2 = Bp / 2;
  const int KG = max(1, kLstmThreads / NB2);
  float* Wc = reinterpret_cast<float*>(smem_raw);                 // [4H][U]
  float* red = Wc + (size_t)H4 * U;                               // [KG][Bp][U]
  float* dh_rec = red + (size_t)KG * Bp * U;                      // [Bp][U]
  float* dc_car = dh_rec + (size_t)Bp * U;                        // [Bp][U]
  X* stage = reinterpret_cast<X*>(dc_car + (size_t)Bp * U);
  for (int idx = threadIdx.x; idx < H4 * U; idx += blockDim.x) {
    const int r = idx / U, jj = idx % U;
    Wc[idx] = jj < nu ? ldf<T>(p.whh, (int64_t)r * H + j0 + jj) : 0.f;
  }
  for (int idx = threadIdx.x; idx < Bp * U; idx += blockDim.x) {
    const int b = idx / U, jj = idx % U;
    const bool in = jj < nu && b < B;
    dh_rec[idx] = (in && p.dhT) ? ldf<T>(p.dhT, (int64_t)b * H + j0 + jj) : 0.f;
    dc_car[idx] = (in && p.dcT) ? ldf<T>(p.dcT, (int64_t)b * H + j0 + jj) : 0.f;
  }
  __syncthreads();
  unsigned int target = 0;
  bool alive = true;
  const int kg = threadIdx.x / NB2, b0 = (threadIdx.x % NB2) * 2;
  const bool active = kg < KG;
  for (int t = p.T - 1; t >= 0 && alive; --t) {
    // ---- phase A: gate gradients of this CTA's units (saved copy [T,B,4H] and k-major exchange copy)
    for (int idx = threadIdx.x; idx < Bp * nu; idx += blockDim.x) {
      const int jj = idx / Bp, b = idx % Bp, j = j0 + jj;
      float dai = 0.f, daf = 0.f, dag = 0.f, dao = 0.f;
      if (b < B) {
        const int64_t gb = ((int64_t)t * H4 + j) * Bp + b, gs = (int64_t)H * Bp;
        const float ig = ldf<T>(p.gates, gb), fg = ldf<T>(p.gates, gb + gs), gg = ldf<T>(p.gates, gb + 2 * gs),
                    og = ldf<T>(p.gates, gb + 3 * gs);
        const float c = p.cs[((int64_t)t * H + j) * Bp + b];
        const float cprev = t > 0 ? p.cs[((int64_t)(t - 1) * H + j) * Bp + b] : ldf<T>(p.c0, (int64_t)b * H + j);
        const float dh = ldf<T>(p.dy, ((int64_t)t * B + b) * H + j) + dh_rec[b * U + jj];
        const float tc = tanhf(c);
        const float dc = dc_car[b * U + jj] + dh * og * (1.f - tc * tc);
        dai = dc * gg * ig * (1.f - ig);
        daf = dc * cprev * fg * (1.f - fg);
        dag = dc * ig * (1.f - gg * gg);
        dao = dh * tc * og * (1.f - og);
        dc_car[b * U + jj] = dc * fg;
      }
      X* dgt = static_cast<X*>(p.dgates) + (int64_t)t * H4 * Bp;       // padding rows get zeros
      dgt[(int64_t)j * Bp + b] = Cvt<X>::from_f(dai);
      dgt[(int64_t)(H + j) * Bp + b] = Cvt<X>::from_f(daf);
      dgt[(int64_t)(2 * H + j) * Bp + b] = Cvt<X>::from_f(dag);
      dgt[(int64_t)(3 * H + j) * Bp + b] = Cvt<X>::from_f(dao);
    }
    target += gridDim.x;
    alive = grid_barrier(p.bar, target);
    if (!alive) break;
    // ---- phase B: dh_{t-1}[b, j] = sum_r dgates[t, b, r] * W_hh[r, j] for this CTA's units j
    float acc[2][U];
    stream_matmul<X, U>(static_cast<const X*>(p.dgates) + (int64_t)t * H4 * Bp, H4, Bp, Wc, stage, p.tileK, kg, KG, b0, active,
                        acc);
    if (active) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float* dst = red + ((size_t)kg * Bp + b0 + rr) * U;
#pragma unroll
        for (int o = 0; o < U; ++o) dst[o] = acc[rr][o];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < Bp * U; idx += blockDim.x) {
      const int b = idx / U, jj = idx % U;
      float s = 0.f;
      for (int q = 0; q < KG; ++q) s += red[((size_t)q * Bp + b) * U + jj];
      dh_rec[idx] = s;
    }
    __syncthreads();
  }
  if (alive) {
    for (int idx = threadIdx.x; idx < B * nu; idx += blockDim.x) {
      const int b = idx / nu, jj = idx % nu;
      stf<T>(p.dh0, (int64_t)b * H + j0 + jj, dh_rec[b * U + jj]);
      stf<T>(p.dc0, (int64_t)b * H + j0 + jj, dc_car[b * U + jj]);
    }
  }
}

// ---- GRU and vanilla RNN --------------------------------------------------------------------------------------------
// Same ownership and exchange as the LSTM kernels with NG gates per unit (3: GRU in the order r, z, n; 1: vanilla RNN).
//   GRU:      r = sigmoid(xr + hr), z = sigmoid(xz + hz), n = tanh(xn + r * (hn + b_hn)), h_t = (1 - z) * n + z * h_{t-1}
//             where x* = x_t.W_ih^T + b_ih (+ b_hh for r and z) comes from the input GEMM and h* = h_{t-1}.W_hh^T
//   vanilla:  h_t = act(x + h_{t-1}.W_hh^T), act = tanh or relu, x including both biases
// (src/operator/rnn_impl.h: GruForwardTraining, VanillaRNNForwardTraining in the reference.)
// Forward shared memory: Wt [H][NG*U], red [KG][Bp][NG*U], hst [Bp][U] (fp32 copy of the CTA's own h), stage.
__host__ __device__ __forceinline__ size_t rnn_align4(size_t floats) { return (floats + 3) & ~(size_t)3; }

template <typename T, typename X, int U, int NG>
__global__ void __launch_bounds__(kLstmThreads) rnn_fwd_kernel(const LstmParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, B = p.B, Bp = p.Bp;
  constexpr int R = NG * U;
  const int j0 = blockIdx.x * U;
  const int nu = min(U, H - j0);
  const int NB2 = Bp / 2;
  const int KG = max(1, kLstmThreads / NB2);
  float* Wt = reinterpret_cast<float*>(smem_raw);                 // [H][R]
  float* red = Wt + (size_t)H * R;                                // [KG][Bp][R]
  float* hst = red + (size_t)KG * Bp * R;                         // [Bp][U]
  // [2][tileK][Bp], on a 16-byte boundary for the cp.async copies (H * R need not be a multiple of four floats)
  X* stage = reinterpret_cast<X*>(Wt + rnn_align4((size_t)H * R + (size_t)KG * Bp * R + (size_t)Bp * U));
  X* hx = static_cast<X*>(p.hbuf);
  for (int idx = threadIdx.x; idx < H * R; idx += blockDim.x) {
    const int k = idx / R, r = idx % R;
    const int g = r / U, jj = r % U;
    Wt[idx] = jj < nu ? ldf<T>(p.whh, (int64_t)(g * H + j0 + jj) * H + k) : 0.f;
  }
  for (int idx = threadIdx.x; idx < Bp * U; idx += blockDim.x) {
    const int b = idx / U, jj = idx % U;
    hst[idx] = (jj < nu && b < B) ? ldf<T>(p.h0, (int64_t)b * H + j0 + jj) : 0.f;
  }
  for (int idx = threadIdx.x; idx < Bp * nu; idx += blockDim.x) {
    const int jj = idx / Bp, b = idx % Bp;
    hx[(int64_t)(j0 + jj) * Bp + b] = Cvt<X>::from_f(b < B ? ldf<T>(p.h0, (int64_t)b * H + j0 + jj) : 0.f);
  }
  unsigned int target = gridDim.x;
  bool alive = grid_barrier(p.bar, target);
  const int kg = threadIdx.x / NB2, b0 = (threadIdx.x % NB2) * 2;
  const bool active = kg < KG;
  for (int t = 0; t < p.T && alive; ++t) {
    const X* hprev = hx + (int64_t)(t & 1) * H * Bp;
    X* hnext = hx + (int64_t)((t + 1) & 1) * H * Bp;
    float xp[2][NG];
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int idx = threadIdx.x + it * kLstmThreads;
      const int jj = idx / Bp, b = idx % Bp;
#pragma unroll
      for (int g = 0; g < NG; ++g)
        xp[it][g] = (idx < Bp * nu && b < B) ? ldf<T>(p.xproj, ((int64_t)t * B + b) * NG * H + g * H + j0 + jj) : 0.f;
    }
    float acc[2][R];
    stream_matmul<X, R>(hprev, H, Bp, Wt, stage, p.tileK, kg, KG, b0, active, acc);
    if (active) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float* dst = red + ((size_t)kg * Bp + b0 + rr) * R;
#pragma unroll
        for (int o = 0; o < R; ++o) dst[o] = acc[rr][o];
      }
    }
    __syncthreads();
    auto update_cell = [&](int idx, const float (&xg)[NG]) {
      const int jj = idx / Bp, b = idx % Bp, j = j0 + jj;
      if (b >= B) { hnext[(int64_t)j * Bp + b] = Cvt<X>::from_f(0.f); return; }
      float a[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        float s = 0.f;
        for (int q = 0; q < KG; ++q) s += red[((size_t)q * Bp + b) * R + g * U + jj];
        a[g] = s;
      }
      float h;
      if constexpr (NG == 3) {
        const float rg = sigmoidf_(xg[0] + a[0]), zg = sigmoidf_(xg[1] + a[1]);
        const float hn = a[2] + ldf<T>(p.bhn, j);
        const float ng = tanhf(xg[2] + rg * hn);
        h = (1.f - zg) * ng + zg * hst[b * U + jj];
        if (p.gates) {
          const int64_t gb = ((int64_t)t * 3 * H + j) * Bp + b, gs = (int64_t)H * Bp;
          stf<T>(p.gates, gb, rg); stf<T>(p.gates, gb + gs, zg); stf<T>(p.gates, gb + 2 * gs, ng);
          stf<T>(p.hnb, ((int64_t)t * H + j) * Bp + b, hn);
        }
      } else {
        const float s = xg[0] + a[0];
        h = p.relu ? fmaxf(s, 0.f) : tanhf(s);
      }
      hst[b * U + jj] = h;
      hnext[(int64_t)j * Bp + b] = Cvt<X>::from_f(h);
      stf<T>(p.y, ((int64_t)t * B + b) * H + j, h);
      if (t == p.T - 1) stf<T>(p.hT, (int64_t)b * H + j, h);
    };
    if ((int)threadIdx.x < Bp * nu) update_cell(threadIdx.x, xp[0]);
    if ((int)threadIdx.x + kLstmThreads < Bp * nu) update_cell(threadIdx.x + kLstmThreads, xp[1]);
    for (int idx = threadIdx.x + 2 * kLstmThreads; idx < Bp * nu; idx += blockDim.x) {
      const int jj = idx / Bp, b = idx % Bp;
      float xg[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) xg[g] = b < B ? ldf<T>(p.xproj, ((int64_t)t * B + b) * NG * H + g * H + j0 + jj) : 0.f;
      update_cell(idx, xg);
    }
    target += gridDim.x;
    alive = grid_barrier(p.bar, target);
  }
}

// Backward shared memory: Wc [NG*H][U], red [KG][Bp][U], dh_rec [Bp][U], dh_dir [Bp][U] (the z * dh term of the GRU),
// stage.  The exchanged array `dgates` [T, NG*H, Bp] holds the gradients w.r.t. the hidden-side products (GRU: dar, daz,
// dan * r); the GRU's gradient w.r.t. the candidate pre-activation itself goes to `dan` for the input-side GEMMs.
template <typename T, typename X, int U, int NG>
__global__ void __launch_bounds__(kLstmThreads) rnn_bwd_kernel(const LstmParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, B = p.B, Bp = p.Bp, K = NG * p.H;
  const int j0 = blockIdx.x * U;
  const int nu = min(U, H - j0);
  const int NB2 = Bp / 2;
  const int KG = max(1, kLstmThreads / NB2);
  float* Wc = reinterpret_cast<float*>(smem_raw);                 // [K][U]
  float* red = Wc + (size_t)K * U;                                // [KG][Bp][U]
  float* dh_rec = red + (size_t)KG * Bp * U;                      // [Bp][U]
  float* dh_dir = dh_rec + (size_t)Bp * U;                        // [Bp][U]
  X* stage = reinterpret_cast<X*>(Wc + rnn_align4((size_t)K * U + (size_t)KG * Bp * U + (size_t)2 * Bp * U));   // 16-byte boundary
  for (int idx = threadIdx.x; idx < K * U; idx += blockDim.x) {
    const int r = idx / U, jj = idx % U;
    Wc[idx] = jj < nu ? ldf<T>(p.whh, (int64_t)r * H + j0 + jj) : 0.f;
  }
  for (int idx = threadIdx.x; idx < Bp * U; idx += blockDim.x) {
    const int b = idx / U, jj = idx % U;
    dh_rec[idx] = (jj < nu && b < B && p.dhT) ? ldf<T>(p.dhT, (int64_t)b * H + j0 + jj) : 0.f;
    dh_dir[idx] = 0.f;
  }
  __syncthreads();
  unsigned int target = 0;
  bool alive = true;
  const int kg = threadIdx.x / NB2, b0 = (threadIdx.x % NB2) * 2;
  const bool active = kg < KG;
  for (int t = p.T - 1; t >= 0 && alive; --t) {
    X* dgt = static_cast<X*>(p.dgates) + (int64_t)t * K * Bp;
    for (int idx = threadIdx.x; idx < Bp * nu; idx += blockDim.x) {
      const int jj = idx / Bp, b = idx % Bp, j = j0 + jj;
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, dn = 0.f, direct = 0.f;
      if (b < B) {
        const float dh = ldf<T>(p.dy, ((int64_t)t * B + b) * H + j) + dh_rec[b * U + jj];
        if constexpr (NG == 3) {
          const int64_t gb = ((int64_t)t * 3 * H + j) * Bp + b, gs = (int64_t)H * Bp;
          const float rg = ldf<T>(p.gates, gb), zg = ldf<T>(p.gates, gb + gs), ng = ldf<T>(p.gates, gb + 2 * gs);
          const float hn = ldf<T>(p.hnb, ((int64_t)t * H + j) * Bp + b);
          const float hp = t > 0 ? ldf<T>(p.y, ((int64_t)(t - 1) * B + b) * H + j) : ldf<T>(p.h0, (int64_t)b * H + j);
          dn = dh * (1.f - zg) * (1.f - ng * ng);
          d1 = dh * (hp - ng) * zg * (1.f - zg);
          d0 = dn * hn * rg * (1.f - rg);
          d2 = dn * rg;
          direct = dh * zg;
        } else {
          const float yv = ldf<T>(p.y, ((int64_t)t * B + b) * H + j);
          d0 = p.relu ? (yv > 0.f ? dh : 0.f) : dh * (1.f - yv * yv);
        }
      }
      dh_dir[b * U + jj] = direct;
      dgt[(int64_t)j * Bp + b] = Cvt<X>::from_f(d0);
      if constexpr (NG == 3) {
        dgt[(int64_t)(H + j) * Bp + b] = Cvt<X>::from_f(d1);
        dgt[(int64_t)(2 * H + j) * Bp + b] = Cvt<X>::from_f(d2);
        stf<T>(p.dan, ((int64_t)t * H + j) * Bp + b, dn);
      }
    }
    target += gridDim.x;
    alive = grid_barrier(p.bar, target);
    if (!alive) break;
    float acc[2][U];
    stream_matmul<X, U>(dgt, K, Bp, Wc, stage, p.tileK, kg, KG, b0, active, acc);
    if (active) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        float* dst = red + ((size_t)kg * Bp + b0 + rr) * U;
#pragma unroll
        for (int o = 0; o < U; ++o) dst[o] = acc[rr][o];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < Bp * U; idx += blockDim.x) {
      const int b = idx / U, jj = idx % U;
      float s = dh_dir[idx];
      for (int q = 0; q < KG; ++q) s += red[((size_t)q * Bp + b) * U + jj];
      dh_rec[idx] = s;
    }
    __syncthreads();
  }
  if (alive) {
    for (int idx = threadIdx.x; idx < B * nu; idx += blockDim.x) {
      const int b = idx / nu, jj = idx % nu;
      stf<T>(p.dh0, (int64_t)b * H + j0 + jj, dh_rec[b * U + jj]);
    }
  }
}

static int lstm_units_per_cta(int H) {
  int u = (H + sm_count() - 1) / sm_count();
  return u < 1 ? 1 : u;
}
static int lstm_bp(int B) { return (B + 7) / 8 * 8; }
// shared memory without the staging buffers
static size_t lstm_fwd_fixed(int B, int H, int U) {
  const int Bp = lstm_bp(B), NB2 = Bp / 2;
  const int KG = kLstmThreads / NB2 > 1 ? kLstmThreads / NB2 : 1;
  return ((size_t)H * 4 * U + (size_t)KG * Bp * 4 * U + (size_t)Bp * U) * sizeof(float);
}
static size_t lstm_bwd_fixed(int B, int H, int U) {
  const int Bp = lstm_bp(B), NB2 = Bp / 2;
  const int KG = kLstmThreads / NB2 > 1 ? kLstmThreads / NB2 : 1;
  return ((size_t)4 * H * U + (size_t)KG * Bp * U + (size_t)2 * Bp * U) * sizeof(float);
}
constexpr size_t kLstmSmemLimit = 220 * 1024;
// rows per staged tile: whatever fits beside the fixed part, at most the whole operand
static int lstm_tile_rows(size_t fixed, int K, int Bp, size_t xsize) {
  if (fixed >= kLstmSmemLimit) return 0;
  const size_t rows = (kLstmSmemLimit - fixed) / (2 * (size_t)Bp * xsize);
  return (int)(rows < (size_t)K ? rows : (size_t)K);
}

template <typename T, typename X, int U>
static int launch_lstm(bool backward, LstmParams& p, cudaStream_t st) {
  const int Bp = lstm_bp(p.B);
  const size_t fixed = backward ? lstm_bwd_fixed(p.B, p.H, U) : lstm_fwd_fixed(p.B, p.H, U);
  const int K = backward ? 4 * p.H : p.H;
  const int tileK = lstm_tile_rows(fixed, K, Bp, sizeof(X));
  if (tileK < kMinTileK && tileK < K) return -4;
  const size_t smem = fixed + (size_t)2 * tileK * Bp * sizeof(X);
  p.tileK = tileK;
  const void* fn = backward ? (const void*)lstm_bwd_kernel<T, X, U> : (const void*)lstm_fwd_kernel<T, X, U>;
  cudaError_t rc = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (rc != cudaSuccess) return (int)rc;
  const int grid = (p.H + U - 1) / U;
  int per_sm = 0;
  rc = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kLstmThreads, smem);
  if (rc != cudaSuccess) return (int)rc;
  if ((int64_t)per_sm * sm_count() < grid) return -4;      // the grid barrier needs every CTA resident
  p.U = U;
  p.Bp = lstm_bp(p.B);
  void* args[] = {&p};
  rc = cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kLstmThreads), args, smem, st);
  return (int)rc;
}

template <typename T, typename X>
static int dispatch_lstm(bool backward, LstmParams& p, cudaStream_t st) {
  const int U = lstm_units_per_cta(p.H);
  switch (U) {
    case 1: return launch_lstm<T, X, 1>(backward, p, st);
    case 2: return launch_lstm<T, X, 2>(backward, p, st);
    case 3: return launch_lstm<T, X, 3>(backward, p, st);
    case 4: return launch_lstm<T, X, 4>(backward, p, st);
    case 5: return launch_lstm<T, X, 5>(backward, p, st);
    case 6: return launch_lstm<T, X, 6>(backward, p, st);
    case 7: return launch_lstm<T, X, 7>(backward, p, st);
    case 8: return launch_lstm<T, X, 8>(backward, p, st);
    default: return -4;
  }
}

static size_t rnn_fwd_fixed(int B, int H, int U, int NG) {
  const int Bp = lstm_bp(B), NB2 = Bp / 2;
  const int KG = kLstmThreads / NB2 > 1 ? kLstmThreads / NB2 : 1;
  return rnn_align4((size_t)H * NG * U + (size_t)KG * Bp * NG * U + (size_t)Bp * U) * sizeof(float);
}
static size_t rnn_bwd_fixed(int B, int H, int U, int NG) {
  const int Bp = lstm_bp(B), NB2 = Bp / 2;
  const int KG = kLstmThreads / NB2 > 1 ? kLstmThreads / NB2 : 1;
  return rnn_align4((size_t)NG * H * U + (size_t)KG * Bp * U + (size_t)2 * Bp * U) * sizeof(float);
}

template <typename T, typename X, int U, int NG>
static int launch_rnn(bool backward, LstmParams& p, cudaStream_t st) {
  const int Bp = lstm_bp(p.B);
  const size_t fixed = backward ? rnn_bwd_fixed(p.B, p.H, U, NG) : rnn_fwd_fixed(p.B, p.H, U, NG);
  const int K = backward ? NG * p.H : p.H;
  const int tileK = lstm_tile_rows(fixed, K, Bp, sizeof(X));
  if (tileK < kMinTileK && tileK < K) return -4;
  const size_t smem = fixed + (size_t)2 * tileK * Bp * sizeof(X);
  p.tileK = tileK;
  const void* fn = backward ? (const void*)rnn_bwd_kernel<T, X, U, NG> : (const void*)rnn_fwd_kernel<T, X, U, NG>;
  cudaError_t rc = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (rc != cudaSuccess) return (int)rc;
  const int grid = (p.H + U - 1) / U;
  int per_sm = 0;
  rc = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kLstmThreads, smem);
  if (rc != cudaSuccess) return (int)rc;
  if ((int64_t)per_sm * sm_count() < grid) return -4;      // the grid barrier needs every CTA resident
  p.U = U;
  p.Bp = Bp;
  void* args[] = {&p};
  rc = cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kLstmThreads), args, smem, st);
  return (int)rc;
}

template <typename T, typename X, int NG>
static int dispatch_rnn(bool backward, LstmParams& p, cudaStream_t st) {
  const int U = lstm_units_per_cta(p.H);
  switch (U) {
    case 1: return launch_rnn<T, X, 1, NG>(backward, p, st);
    case 2: return launch_rnn<T, X, 2, NG>(backward, p, st);
    case 3: return launch_rnn<T, X, 3, NG>(backward, p, st);
    case 4: return launch_rnn<T, X, 4, NG>(backward, p, st);
    case 5: return launch_rnn<T, X, 5, NG>(backward, p, st);
    case 6: return launch_rnn<T, X, 6, NG>(backward, p, st);
    case 7: return launch_rnn<T, X, 7, NG>(backward, p, st);
    case 8: return launch_rnn<T, X, 8, NG>(backward, p, st);
    default: return -4;
  }
}

template <int NG>
static int dispatch_rnn_dtype(int dtype, bool backward, LstmParams& p, cudaStream_t st) {
  if (dtype == kF32) return dispatch_rnn<float, float, NG>(backward, p, st);
  if (dtype == kF16) return dispatch_rnn<__half, __half, NG>(backward, p, st);
  if (dtype == kBF16) return dispatch_rnn<__nv_bfloat16, __nv_bfloat16, NG>(backward, p, st);
  return -1;
}

}  // namespace mxb

using namespace mxb;

// 1 when the persistent kernels can run this shape on the current device (shared-memory and residency limits).
MXB_EXPORT int mxb_lstm_supported(int B, int H) {
  if (B < 1 || H < 1 || lstm_bp(B) > 2 * kLstmThreads) return 0;
  const int U = lstm_units_per_cta(H);
  if (U > 8) return 0;
  const int Bp = lstm_bp(B);
  const int tf = lstm_tile_rows(lstm_fwd_fixed(B, H, U), H, Bp, 4), tb = lstm_tile_rows(lstm_bwd_fixed(B, H, U), 4 * H, Bp, 4);
  return (tf >= kMinTileK || tf >= H) && (tb >= kMinTileK || tb >= 4 * H);
}

// Bytes of the forward exchange buffer `hbuf` for (B, H): [2][H][Bp] floats covers every element type.
MXB_EXPORT int64_t mxb_lstm_exchange_bytes(int B, int H) { return (int64_t)2 * H * lstm_bp(B) * 4; }
// Row length of the k-major arrays (`gates` [T,4H,Bp], `cs` [T,H,Bp], `dgates` [T,4H,Bp]).
MXB_EXPORT int mxb_lstm_bp(int B) { return lstm_bp(B); }

// `bar`: two zero-initialised 32-bit words (arrival counter, error flag); after the kernel bar[1] != 0 means a barrier
// timed out and the outputs are incomplete.  `hbuf`: mxb_lstm_exchange_bytes(B, H) bytes of scratch.
MXB_EXPORT int mxb_lstm_forward(int dtype, const void* xproj, const void* whh, const void* h0, const void* c0, void* y,
                                void* hT, void* cT, void* gates, float* cs, void* hbuf, unsigned int* bar, int T, int B,
                                int H, void* stream) {
  if (!mxb_lstm_supported(B, H) || T < 1) return -4;
  LstmParams p{};
  p.xproj = xproj; p.whh = whh; p.h0 = h0; p.c0 = c0; p.y = y; p.hT = hT; p.cT = cT; p.gates = gates; p.cs = cs;
  p.hbuf = hbuf; p.bar = bar; p.T = T; p.B = B; p.H = H;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) return dispatch_lstm<float, float>(false, p, st);
  if (dtype == kF16) return dispatch_lstm<__half, __half>(false, p, st);
  if (dtype == kBF16) return dispatch_lstm<__nv_bfloat16, __nv_bfloat16>(false, p, st);
  return -1;
}

MXB_EXPORT int mxb_lstm_backward(int dtype, const void* dy, const void* dhT, const void* dcT, const void* gates,
                                 const float* cs, const void* c0, const void* whh, void* dgates, void* dh0, void* dc0,
                                 unsigned int* bar, int T, int B, int H, void* stream) {
  if (!mxb_lstm_supported(B, H) || T < 1) return -4;
  LstmParams p{};
  p.dy = dy; p.dhT = dhT; p.dcT = dcT; p.gates = const_cast<void*>(gates); p.cs = const_cast<float*>(cs); p.c0 = c0;
  p.whh = whh; p.dgates = dgates; p.dh0 = dh0; p.dc0 = dc0; p.bar = bar; p.T = T; p.B = B; p.H = H;
  cudaStream_t st = (cudaStream_t)stream;
  // the gate gradients cross CTAs in the model type: the copy saved for the weight-gradient GEMMs has that type too
  if (dtype == kF32) return dispatch_lstm<float, float>(true, p, st);
  if (dtype == kF16) return dispatch_lstm<__half, __half>(true, p, st);
  if (dtype == kBF16) return dispatch_lstm<__nv_bfloat16, __nv_bfloat16>(true, p, st);
  return -1;
}

// GRU (mode 0), vanilla RNN with tanh (1) or relu (2).  `xproj` [T, B, NG*H] holds x.W_ih^T + b_ih, plus b_hh except for
// the GRU's candidate gate whose hidden-side bias is `bhn` [H].  `gates` [T, 3H, Bp] and `hnb` [T, H, Bp] are written
// for the GRU when non-null (training).  Shapes accepted: mxb_lstm_supported(B, H).
MXB_EXPORT int mxb_rnn_forward(int dtype, int mode, const void* xproj, const void* whh, const void* bhn, const void* h0,
                               void* y, void* hT, void* gates, void* hnb, void* hbuf, unsigned int* bar, int T, int B, int H,
                               void* stream) {
  if (!mxb_lstm_supported(B, H) || T < 1 || mode < 0 || mode > 2) return -4;
  if (mode == 0 && bhn == nullptr) return -2;
  LstmParams p{};
  p.xproj = xproj; p.whh = whh; p.bhn = bhn; p.h0 = h0; p.y = y; p.hT = hT; p.gates = gates; p.hnb = hnb; p.hbuf = hbuf;
  p.bar = bar; p.T = T; p.B = B; p.H = H; p.relu = mode == 2;
  cudaStream_t st = (cudaStream_t)stream;
  return mode == 0 ? dispatch_rnn_dtype<3>(dtype, false, p, st) : dispatch_rnn_dtype<1>(dtype, false, p, st);
}

// `dgates` [T, NG*H, Bp]: gradients w.r.t. the hidden-side products (output; also the exchanged operand).  GRU only:
// `gates`, `hnb` from the forward pass, `dan` [T, H, Bp] receives the gradient w.r.t. the candidate pre-activation.
MXB_EXPORT int mxb_rnn_backward(int dtype, int mode, const void* dy, const void* dhT, const void* gates, const void* hnb,
                                const void* y, const void* h0, const void* whh, void* dgates, void* dan, void* dh0,
                                unsigned int* bar, int T, int B, int H, void* stream) {
  if (!mxb_lstm_supported(B, H) || T < 1 || mode < 0 || mode > 2) return -4;
  if (mode == 0 && (gates == nullptr || hnb == nullptr || dan == nullptr)) return -2;
  LstmParams p{};
  p.dy = dy; p.dhT = dhT; p.gates = const_cast<void*>(gates); p.hnb = const_cast<void*>(hnb); p.y = const_cast<void*>(y);
  p.h0 = h0; p.whh = whh; p.dgates = dgates; p.dan = dan; p.dh0 = dh0; p.bar = bar; p.T = T; p.B = B; p.H = H;
  p.relu = mode == 2;
  cudaStream_t st = (cudaStream_t)stream;
  return mode == 0 ? dispatch_rnn_dtype<3>(dtype, true, p, st) : dispatch_rnn_dtype<1>(dtype, true, p, st);
}

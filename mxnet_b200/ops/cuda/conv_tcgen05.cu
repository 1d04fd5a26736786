// Stride-1 NHWC convolution (forward and data gradient) as an implicit GEMM on tcgen05 tensor cores, for sm_100a.
//
//   Y[n, h, w, co] = act( sum_{r, s, c} X[n, h + off_h + r*step_h, w + off_w + s*step_w, c] * Wt[co, r, s, c]
//                         + bias[co] + res[n, h, w, co] )
//
// Reference behaviour: src/operator/nn/convolution.cu / cudnn_ops (cuDNN fprop / dgrad on NHWC tensors, with
// im2col + GEMM as the generic path, src/operator/nn/im2col.cuh).  Here no im2col buffer exists: a tile of 128
// output pixels is a small box (bw x bh x bnb) of the (w, h, n) pixel space, and for every filter tap the TMA
// engine loads that box of the input, shifted by the tap offset, as a 4-D tile {64 channels, bw, bh, bnb}; positions
// outside the image read the fill value 0, which is the zero padding.  The box lands in shared memory as 128 rows of
// 128 bytes with the 128-byte swizzle, exactly the K-major operand of the GEMM kernel, so the contraction loop is a
// GEMM whose k-steps run over (tap, channel chunk).  The weights stay in their stored layout [Cout, R, S, Cin]:
//   forward        : B is K-major   (k = input channel, contiguous), box {64 c, 1 tap, BN co}
//   data gradient  : B is MN-major  (n = input channel, contiguous; k = output channel), box {64 c, 1 tap, 64 co};
//                    the tap offsets are negated, which is the 180-degree rotation of the filter.
// The epilogue maps accumulator rows back to pixels, adds bias and residual, applies ReLU, stores, and can
// accumulate per-channel sum / sum of squares of the fp32 results (the BatchNorm batch statistics of the layer that
// follows) so that the normalisation does not have to read the tensor again to reduce it.
//
// Roles, ring, TMEM double buffering and the bounded waits are those of the GEMM kernel (gemm_tcgen05.cu).
#include <cstdlib>

#include "tcgen05.cuh"

namespace mxb {

constexpr int CBM = 128, CBK = 64, CUMMA_K = 16;
constexpr int kConvThreads = 192;          // weight-gradient kernel: producer, MMA, 4 epilogue warps
constexpr int kIgemmThreads = 320;         // forward / data-gradient kernel: producer, MMA, 8 epilogue warps
constexpr uint32_t CA_BYTES = CBM * CBK * 2;
constexpr int kConvMaxStages = 8;
constexpr uint32_t kSmemLimit = 232448;    // 227 KB per CTA
constexpr uint32_t kStgBytes = 8 * 2048;           // per epilogue warp: 32 rows x 64 bytes staged for the TMA store

template <int BN> struct ConvCfg {
  static constexpr uint32_t B_BYTES = BN * CBK * 2;
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr uint32_t STAT_BYTES = 4 * 2 * BN * 4;     // [TMEM lane quarter][sum | sumsq][BN] floats
  static constexpr uint32_t SMEM_BYTES = STAGES * (CA_BYTES + B_BYTES) + STAT_BYTES + 1024 /*alignment*/ + 512 /*barriers*/;
  // forward / data-gradient kernel: everything except the operand buffers
  static constexpr uint32_t FIXED_BYTES = STAT_BYTES + kStgBytes + 512;
  static constexpr uint32_t OPERAND_BUDGET = kSmemLimit - 1024 - FIXED_BYTES;
};

struct ConvGeom {
  int N, Ho, Wo;                         // output pixel space
  int NC, KC;                            // output channels of this launch (GEMM N), reduction channels (per tap)
  int R, S;
  int off_h, step_h, off_w, step_w;      // input row of tap r for output row h: h * str_h + off_h + r * step_h
  int str_h, str_w;                      // convolution stride (1 except for the strided forward convolution)
  int bw, bh, bnb;                       // pixel box, bw * bh * bnb = 128
  int tiles_w, tiles_h, tiles_nb;
  int ldy;                               // channel pitch of Y and of the residual, in elements
  int b_mn;                              // 0: weights K-major (forward), 1: MN-major (data gradient)
  int act;                               // 0 none, 1 ReLU
  int bf16;
  int stages;                            // depth of the operand ring
  int stationary;                        // 1: all weight slices of a column tile stay in shared memory, the ring holds A only
  int log_bw, log_bh;                    // the pixel box sides are powers of two
  FastDiv fd_tiles_m, fd_tiles_w, fd_tiles_h;
};

// tile index -> (column tile, first pixel of the row tile), without hardware division
struct TilePos {
  int tile_n, w0, h0, n0;
};
__device__ __forceinline__ TilePos tile_pos(int tile, const ConvGeom& g) {
  uint32_t tn, tm, rest, tw, tnb, th;
  fd_divmod((uint32_t)tile, g.fd_tiles_m, &tn, &tm);
  fd_divmod(tm, g.fd_tiles_w, &rest, &tw);
  fd_divmod(rest, g.fd_tiles_h, &tnb, &th);
  TilePos p;
  p.tile_n = (int)tn;
  p.w0 = (int)tw << g.log_bw;
  p.h0 = (int)th << g.log_bh;
  p.n0 = (int)tnb * g.bnb;
  return p;
}

// Shared-memory carve-up (after 1024-byte alignment):
//   [A ring: stages x 16 KB][B: ring of stages x B_BYTES, or taps*kchunks resident slices][store staging][stat][barriers]
template <typename T, int BN>
__global__ void __launch_bounds__(kIgemmThreads, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_y, const T* __restrict__ bias, const T* __restrict__ res, float* __restrict__ stat_partial,
                  const ConvGeom g, int* __restrict__ error_flag, long long* __restrict__ prof) {
  using Cfg = ConvCfg<BN>;
  constexpr uint32_t B_BYTES = Cfg::B_BYTES;
  // optional cycle accounting of CTA 0 (prof != nullptr): where each role spends its time
  const bool profiling = prof != nullptr && blockIdx.x == 0;
  long long pc[6] = {0, 0, 0, 0, 0, 0};
  const long long t_begin = clock64();
  long long t_last = t_begin;
  // attribute the cycles since the previous mark to bucket b (a full partition of a role's time)
#define MXB_PROF_MARK(b)                 \
  if (profiling) {                       \
    const long long t_now = clock64();   \
    pc[b] += t_now - t_last;             \
    t_last = t_now;                      \
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int kchunks = (g.KC + CBK - 1) / CBK;
  const int num_k = g.R * g.S * kchunks;
  const int STAGES = g.stages;
  const uint32_t b_region = (g.stationary ? (uint32_t)num_k : (uint32_t)STAGES) * B_BYTES;
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * CA_BYTES;
  uint8_t* sstg = sB + b_region;                                   // 1024-byte aligned: both regions before it are
  float* sstat = reinterpret_cast<float*>(sB + b_region + kStgBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + b_region + kStgBytes + Cfg::STAT_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + kConvMaxStages;
  uint64_t* acc_full = bars + 2 * kConvMaxStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* w_full = acc_empty + 2;       // resident weights loaded
  uint64_t* w_free = w_full + 1;          // resident weights no longer read by any MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_it = abort_flag + 1;
  volatile int* consumed_it = abort_flag + 2;
  volatile int* w_issued = abort_flag + 3;      // weight loads issued / observed complete
  volatile int* w_consumed = abort_flag + 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = g.tiles_w * g.tiles_h * g.tiles_nb;
  const int tiles_n = (g.NC + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  constexpr uint32_t kTmemCols = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kConvMaxStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    mbar_init(w_full, 1);
    mbar_init(w_free, 1);
    *abort_flag = 0;
    *issued_it = 0;
    *consumed_it = 0;
    *w_issued = 0;
    *w_consumed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 4 * 2 * BN; i += kIgemmThreads) sstat[i] = 0.f;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // Producer and MMA warps: the whole warp walks the loops (waits, ring counters, descriptor arithmetic), so every value
  // is warp-uniform, and lane 0 alone issues the TMA / tcgen05 instructions.  Ring position and parity are running
  // counters (no divisions) and descriptors advance by additions: the per-k-step instruction count of these two warps
  // bounds narrow tiles.
  if (warp == 0) {
    int it = 0, st = 0, cur_tn = -1, wloads = 0;
    uint32_t ph = 0;
    const uint32_t stage_bytes = g.stationary ? CA_BYTES : CA_BYTES + B_BYTES;
    const int taps = g.R * g.S;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok && !*abort_flag; tile += gridDim.x) {
      const TilePos tp = tile_pos(tile, g);
      const int tile_n = tp.tile_n, w0 = tp.w0, h0 = tp.h0, n0 = tp.n0;
      if (g.stationary && tile_n != cur_tn) {
        // a new column tile: (re)load all of its weight slices, once the MMAs of the previous column tile are done
        if (wloads > 0 && !mbar_wait_warp(w_free, (uint32_t)(wloads - 1) & 1u)) { *abort_flag = 1; break; }
        if (lane == 0) {
          mbar_expect_tx(w_full, (uint32_t)num_k * B_BYTES);
          for (int tap = 0; tap < taps; ++tap) {
            for (int kc = 0; kc < kchunks; ++kc) {
              uint8_t* dst = sB + (size_t)(tap * kchunks + kc) * B_BYTES;
              if (!g.b_mn) {
                tma_load_3d(dst, &map_w, kc * CBK, tap, tile_n * BN, w_full);
              } else {
#pragma unroll
                for (int c = 0; c < BN / 64; ++c)
                  tma_load_3d(dst + c * kMnChunkBytes, &map_w, tile_n * BN + c * 64, tap, kc * CBK, w_full);
              }
            }
          }
        }
        ++wloads;
        if (lane == 0) *w_issued = wloads;
        cur_tn = tile_n;
        __syncwarp();
      }
      int tap = 0;
      for (int r = 0; r < g.R && ok; ++r) {
        const int ih = h0 * g.str_h + g.off_h + r * g.step_h;
        for (int s = 0; s < g.S && ok; ++s, ++tap) {
          const int iw = w0 * g.str_w + g.off_w + s * g.step_w;
          for (int kc = 0; kc < kchunks; ++kc) {
            MXB_PROF_MARK(4)                                       // loop overhead since the previous k-step
            if (!mbar_wait_warp(&empty[st], ph ^ 1u)) { *abort_flag = 1; ok = false; break; }
            MXB_PROF_MARK(0)                                       // waiting for a free stage
            if (lane == 0) {
              mbar_expect_tx(&full[st], stage_bytes);
              MXB_PROF_MARK(2)
              tma_load_4d(sA + st * CA_BYTES, &map_x, kc * CBK, iw, ih, n0, &full[st]);
              if (!g.stationary) {
                if (!g.b_mn) {
                  tma_load_3d(sB + st * B_BYTES, &map_w, kc * CBK, tap, tile_n * BN, &full[st]);
                } else {
#pragma unroll
                  for (int c = 0; c < BN / 64; ++c)
                    tma_load_3d(sB + st * B_BYTES + c * kMnChunkBytes, &map_w, tile_n * BN + c * 64, tap, kc * CBK, &full[st]);
                }
              }
              MXB_PROF_MARK(3)
            }
            __syncwarp();
            ++it;
            if (++st == STAGES) { st = 0; ph ^= 1u; }
          }
        }
      }
    }
    if (lane == 0) {
      *issued_it = it;
      if (profiling) { prof[0] = pc[0]; prof[1] = clock64() - t_begin; prof[2] = it; prof[9] = pc[2]; prof[10] = pc[3]; prof[13] = pc[4]; }
    }
  } else if (warp == 1) {
    const uint32_t idesc = make_idesc(g.bf16, BN, 0, g.b_mn);
    const uint64_t b_step = g.b_mn ? (16 * 128) >> 4 : 2;
    // descriptors of stage 0 / slice 0; the start-address field (16-byte units, 14 bits) takes plain additions
    const uint64_t adesc0 = make_desc(smem_u32(sA));
    const uint64_t bdesc0 = g.b_mn ? make_desc_mn(smem_u32(sB)) : make_desc(smem_u32(sB));
    int it = 0, st = 0, t = 0, cur_tn = -1, wloads = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok && !*abort_flag; tile += gridDim.x, ++t) {
      const int tile_n = (int)fd_div((uint32_t)tile, g.fd_tiles_m);
      const int buf = t & 1;
      if (g.stationary && tile_n != cur_tn) {
        if (!mbar_wait_warp(w_full, (uint32_t)wloads & 1u)) { *abort_flag = 1; break; }
        ++wloads;
        if (lane == 0) *w_consumed = wloads;
        cur_tn = tile_n;
      }
      MXB_PROF_MARK(4)
      if (!mbar_wait_warp(&acc_empty[buf], (((uint32_t)t >> 1) & 1u) ^ 1u)) { *abort_flag = 1; break; }
      MXB_PROF_MARK(1)                                             // waiting for a drained accumulator
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
      for (int kt = 0; kt < num_k; ++kt) {
        MXB_PROF_MARK(4)                                           // loop overhead since the previous k-step
        if (!mbar_wait_warp(&full[st], ph)) { *abort_flag = 1; ok = false; break; }
        MXB_PROF_MARK(0)                                           // waiting for operands
        const uint64_t adesc = adesc0 + (uint64_t)(st * (int)(CA_BYTES >> 4));
        const uint64_t bdesc = bdesc0 + (uint64_t)((g.stationary ? kt : st) * (int)(B_BYTES >> 4));
        if (lane == 0) {
          umma(tmem_d, adesc, bdesc, idesc, kt > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < CBK / CUMMA_K; ++k)
            umma(tmem_d, adesc + 2 * (uint64_t)k, bdesc + b_step * (uint64_t)k, idesc, 1u);
          MXB_PROF_MARK(2)
          umma_commit(&empty[st]);
          MXB_PROF_MARK(3)
        }
        __syncwarp();
        ++it;
        if (++st == STAGES) { st = 0; ph ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) {
        umma_commit(&acc_full[buf]);
        if (g.stationary) {
          const int next = tile + gridDim.x;
          if (next < num_tiles && (int)fd_div((uint32_t)next, g.fd_tiles_m) != tile_n) umma_commit(w_free);   // last tile of this column tile
        }
      }
      __syncwarp();
    }
    if (lane == 0) {
      *consumed_it = it;
      if (profiling) { prof[3] = pc[0]; prof[4] = pc[1]; prof[5] = clock64() - t_begin; prof[6] = t; prof[11] = pc[2]; prof[12] = pc[3]; prof[14] = pc[4]; }
    }
  } else {
    // Epilogue warps 2..9.  A warp may only read the TMEM lanes of its quarter (warp index modulo 4); the two warps of
    // a quarter split the tile's columns in halves.
    const int q = warp & 3, half = (warp - 2) >> 2;
    float* my_sum = sstat + (q * 2 + 0) * BN;
    float* my_sq = sstat + (q * 2 + 1) * BN;
    uint8_t* stg = sstg + (warp - 2) * 2048;                        // this warp's staging tile: 32 rows x 64 bytes
    float* scr = reinterpret_cast<float*>(stg);                     // the same bytes as a 32 x 16 float transpose tile
    constexpr int HALF_COLS = BN / 2;
    // the 32 accumulator rows of this warp are a sub-box (sbw x sbh x sbn) of the tile's pixel box
    const int r0 = q * 32;
    const int sub_w = r0 & (g.bw - 1), sub_h = (r0 >> g.log_bw) & (g.bh - 1), sub_n = r0 >> (g.log_bw + g.log_bh);
    int t = 0, stat_tile_n = -1;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      const TilePos tp = tile_pos(tile, g);
      const int tile_n = tp.tile_n;
      const int buf = t & 1;
      long long te0 = 0;
      if (profiling) te0 = clock64();
      const bool ready = mbar_wait(&acc_full[buf], ((uint32_t)t >> 1) & 1u);
      if (!ready) *abort_flag = 1;
      if (!ready || *abort_flag) break;
      if (profiling) pc[0] += clock64() - te0;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (stat_partial != nullptr && stat_tile_n != tile_n) {
        if (stat_tile_n >= 0) {
          float* prow = stat_partial + (size_t)(blockIdx.x * 4 + q) * 2 * g.NC;
          for (int c = half * HALF_COLS + lane; c < (half + 1) * HALF_COLS; c += 32) {
            const int col = stat_tile_n * BN + c;
            if (col < g.NC) { prow[col] = my_sum[c]; prow[g.NC + col] = my_sq[c]; }
            my_sum[c] = 0.f;
            my_sq[c] = 0.f;
          }
        }
        stat_tile_n = tile_n;
      }
      const int i = q * 32 + lane;
      const int wl = i & (g.bw - 1), hl = (i >> g.log_bw) & (g.bh - 1), nl = i >> (g.log_bw + g.log_bh);
      const int ow = tp.w0 + wl, oh = tp.h0 + hl, on = tp.n0 + nl;
      const bool row_ok = ow < g.Wo && oh < g.Ho && on < g.N;
      const size_t pix = ((size_t)on * g.Ho + oh) * g.Wo + ow;
      const bool bias_vec = bias != nullptr && ((reinterpret_cast<uintptr_t>(bias) & 15) == 0);
      const bool row_vec = (g.ldy % 8) == 0;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      uint32_t rr[32];
      tmem_ld32(taddr + (uint32_t)(half * HALF_COLS), rr);
#pragma unroll 1
      for (int c0 = half * HALF_COLS; c0 < (half + 1) * HALF_COLS; c0 += 32) {
        const int col0 = tile_n * BN + c0;
        const bool full_cols = col0 + 32 <= g.NC;
        float bv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) bv[j] = 0.f;
        if (bias != nullptr && col0 < g.NC) {
          if (bias_vec && full_cols) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const Vec16<T> b = ld16(bias + col0 + v * 8);
#pragma unroll
              for (int j = 0; j < 8; ++j) bv[v * 8 + j] = Cvt<T>::to_f(b.v[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < g.NC) bv[j] = Cvt<T>::to_f(bias[col0 + j]);
          }
        }
        if (res != nullptr && row_ok && col0 < g.NC) {
          const T* rrow = res + pix * g.ldy + col0;
          if (full_cols && row_vec) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const Vec16<T> b = ld16(rrow + v * 8);
#pragma unroll
              for (int j = 0; j < 8; ++j) bv[v * 8 + j] += Cvt<T>::to_f(b.v[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < g.NC) bv[j] += Cvt<T>::to_f(rrow[j]);
          }
        }
        tmem_wait_ld32(rr);
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float x = __uint_as_float(rr[j]) + bv[j];
          if (g.act == 1) x = fmaxf(x, 0.f);
          f[j] = x;
        }
        // the next 32 columns travel from TMEM while these are converted and stored
        if (c0 + 32 < (half + 1) * HALF_COLS) tmem_ld32(taddr + (uint32_t)(c0 + 32), rr);
        // the staging tile is free once the previous store of this warp has read it
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        if (stat_partial != nullptr) {
          // column sums over the warp's 32 rows, 16 columns at a time through the staging bytes as a 32 x 16 float
          // tile (column index xor-ed with the row to spread the banks): thread (row) writes its 16 values, then lane
          // l adds column (l & 15) over rows 16*(l >> 4) .. +15
#pragma unroll
          for (int hcol = 0; hcol < 2; ++hcol) {
#pragma unroll
            for (int j = 0; j < 16; ++j) scr[lane * 16 + (j ^ (lane & 15))] = row_ok ? f[hcol * 16 + j] : 0.f;
            __syncwarp();
            float sa = 0.f, sb = 0.f;
            const int cc = lane & 15, rb = (lane >> 4) * 16;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
              const float v = scr[(rb + r) * 16 + (cc ^ r)];
              sa += v;
              sb = fmaf(v, v, sb);
            }
            sa += __shfl_xor_sync(0xffffffffu, sa, 16);
            sb += __shfl_xor_sync(0xffffffffu, sb, 16);
            if (lane < 16) {
              my_sum[c0 + hcol * 16 + lane] += sa;
              my_sq[c0 + hcol * 16 + lane] += sb;
            }
            __syncwarp();
          }
        }
        if (col0 < g.NC) {
          // this row's 32 values as four 16-byte pieces in the 64-byte-swizzled layout of the store's tensor map
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            Vec16<T> o;
#pragma unroll
            for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(f[v * 8 + j]);
            st16(reinterpret_cast<T*>(stg + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)), o);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&map_y, stg, col0, tp.w0 + sub_w, tp.h0 + sub_h, tp.n0 + sub_n);
            tma_store_commit();
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (lane == 0) tma_store_wait_all();            // the staging tile must outlive the last store
    if (profiling && warp == 2 && lane == 0) { prof[7] = pc[0]; prof[8] = clock64() - t_begin; }
    if (stat_partial != nullptr && stat_tile_n >= 0) {
      __syncwarp();
      float* prow = stat_partial + (size_t)(blockIdx.x * 4 + q) * 2 * g.NC;
      for (int c = half * HALF_COLS + lane; c < (half + 1) * HALF_COLS; c += 32) {
        const int col = stat_tile_n * BN + c;
        if (col < g.NC) { prow[col] = my_sum[c]; prow[g.NC + col] = my_sq[c]; }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    // gave up somewhere: wait (bounded) for bulk copies that were issued but never consumed before the shared
    // memory is released
    for (int it = *consumed_it; it < *issued_it; ++it) mbar_wait(&full[it % STAGES], (uint32_t)(it / STAGES) & 1u);
    for (int k = *w_consumed; k < *w_issued; ++k) mbar_wait(w_full, (uint32_t)k & 1u);
    if (error_flag) atomicExch(error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace mxb

namespace mxb {

// Pixel box (bw, bh, bnb) with bw * bh * bnb = total that covers the (Wo, Ho, N) space with the fewest tiles;
// among equals the widest box wins (longer contiguous runs in memory).
static void choose_box(int Wo, int Ho, int N, int total, int* bw, int* bh, int* bnb) {
  long best = -1;
  for (int w = total; w >= 1; w >>= 1) {
    for (int h = total / w; h >= 1; h >>= 1) {
      const int nb = total / (w * h);
      if (w > 256 || h > 256 || nb > 256) continue;
      const long tiles = (long)((Wo + w - 1) / w) * ((Ho + h - 1) / h) * ((N + nb - 1) / nb);
      if (best < 0 || tiles < best) { best = tiles; *bw = w; *bh = h; *bnb = nb; }
    }
  }
}

// NHWC activation tensor [N, H, W, C] as a 4-D map {C, W, H, N}; box {64, bw, bh, bnb}; 128-byte swizzle; zero fill.
// (sh, sw) > 1 describes every sh-th row and sw-th column of the stored tensor (the input of a strided 1x1 convolution):
// a view of ceil(H / sh) x ceil(W / sw) pixels with the strides multiplied accordingly.
// (th, tw) > 1 are traversal strides: a box still delivers bw x bh pixels, but every tw-th column and th-th row
// starting at the box origin, which may have any parity (the input of a strided convolution with a filter larger than
// 1x1, whose taps shift the origin by single pixels).
static int make_map_nhwc(CUtensorMap* map, const void* base, int bf16, int N, int H, int W, int C, int bw, int bh, int bnb,
                         int sh = 1, int sw = 1, int th = 1, int tw = 1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  if ((bw - 1) * tw + 1 > 256 || (bh - 1) * th + 1 > 256) return -12;      // a box spans at most 256 elements per axis
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)((W + sw - 1) / sw), (cuuint64_t)((H + sh - 1) / sh), (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)sw * C * 2, (cuuint64_t)sh * W * C * 2, (cuuint64_t)H * W * C * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)((bw - 1) * tw + 1), (cuuint32_t)((bh - 1) * th + 1), (cuuint32_t)bnb};
  cuuint32_t estr[4] = {1, (cuuint32_t)tw, (cuuint32_t)th, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// Output tensor [N, Ho, Wo, C] for the epilogue's stores: box {32 channels, sw, sh, sn} (32 pixels), 64-byte swizzle.
static int make_map_store(CUtensorMap* map, const void* base, int bf16, int N, int H, int W, int C, int sw, int sh, int sn,
                          int ph = 1, int pw = 1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  // (ph, pw) > 1: the stores go to every ph-th row and pw-th column of the stored tensor (the data gradient of a
  // strided 1x1 convolution, whose other positions are zero)
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)((W + pw - 1) / pw), (cuuint64_t)((H + ph - 1) / ph), (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)pw * C * 2, (cuuint64_t)ph * W * C * 2, (cuuint64_t)H * W * C * 2};
  cuuint32_t box[4] = {32, (cuuint32_t)sw, (cuuint32_t)sh, (cuuint32_t)sn};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// Filter [Cout, taps, Cin] as a 3-D map {Cin, taps, Cout}; box {64, 1, box_co}.
static int make_map_filter(CUtensorMap* map, const void* base, int bf16, int Cout, int taps, int Cin, int box_co) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {(cuuint64_t)Cin, (cuuint64_t)taps, (cuuint64_t)Cout};
  cuuint64_t strides[2] = {(cuuint64_t)Cin * 2, (cuuint64_t)taps * Cin * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_co};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// Device buffer of 16 cycle counters filled by CTA 0 of the next launches (null = off), see mxb_conv_set_profile.
static long long* g_conv_prof = nullptr;

template <typename T, int BN>
static int launch_conv(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& my, const void* bias, const void* res,
                       float* stats, ConvGeom g, int* error_flag, cudaStream_t st) {
  using Cfg = ConvCfg<BN>;
  static unsigned long long attr_seen = 0;
  if (first_on_device(&attr_seen)) {
    cudaError_t rc = cudaFuncSetAttribute(conv_igemm_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (rc != cudaSuccess) return (int)rc;
  }
  // Operand buffers: when all weight slices of one column tile fit beside at least four A stages they are loaded once
  // per column tile and stay resident (the ring then carries activations only); otherwise A and B share the ring.
  const int num_k = g.R * g.S * ((g.KC + CBK - 1) / CBK);
  const long wbytes = (long)num_k * Cfg::B_BYTES;
  const long a_stages = ((long)Cfg::OPERAND_BUDGET - wbytes) / CA_BYTES;
  static const bool allow_resident = [] {
    const char* e = getenv("MXNET_B200_CONV_RESIDENT_WEIGHTS");
    return !(e && e[0] == '0');
  }();
  if (allow_resident && a_stages >= 4) {
    g.stationary = 1;
    g.stages = a_stages > kConvMaxStages ? kConvMaxStages : (int)a_stages;
  } else {
    g.stationary = 0;
    g.stages = Cfg::OPERAND_BUDGET / (CA_BYTES + Cfg::B_BYTES);
    if (g.stages > kConvMaxStages) g.stages = kConvMaxStages;
  }
  const uint32_t b_region = (g.stationary ? (uint32_t)num_k : (uint32_t)g.stages) * Cfg::B_BYTES;
  const uint32_t smem_bytes = g.stages * CA_BYTES + b_region + Cfg::FIXED_BYTES + 1024;
  if (smem_bytes > kSmemLimit) return -4;
  const long tiles = (long)g.tiles_w * g.tiles_h * g.tiles_nb * ((g.NC + BN - 1) / BN);
  const int grid = tiles < sm_count() ? (int)tiles : sm_count();
  if (stats) {
    cudaError_t rc = cudaMemsetAsync(stats, 0, (size_t)sm_count() * 4 * 2 * g.NC * sizeof(float), st);
    if (rc != cudaSuccess) return (int)rc;
  }
  conv_igemm_kernel<T, BN><<<grid, kIgemmThreads, smem_bytes, st>>>(mx, mw, my, (const T*)bias, (const T*)res, stats, g,
                                                                    error_flag, g_conv_prof);
  return (int)cudaGetLastError();
}

static int conv_pick_bn(long tiles_m, int NC) {
  if (NC <= 64) return 64;
  if (NC <= 128) return 128;
  if (tiles_m * ((NC + 255) / 256) >= sm_count()) return 256;
  return 128;
}

// Shared by the forward and data-gradient entry points.  `in` is [N, Hi, Wi, KC], the result [N, Ho, Wo, NC].
static int conv_run(int dtype, const void* in, const void* w, void* out, const void* bias, const void* res, float* stats,
                    int N, int Hi, int Wi, int KC, int Ho, int Wo, int NC, int R, int S, int off_h, int step_h, int off_w,
                    int step_w, int w_cout, int w_cin, int b_mn, int act, int* error_flag, cudaStream_t st, int in_sh = 1,
                    int in_sw = 1, int out_sh = 1, int out_sw = 1, int out_full_h = 0, int out_full_w = 0, int str_h = 1,
                    int str_w = 1) {
  if (dtype != kF16 && dtype != kBF16) return -1;
  if (N < 1 || Hi < 1 || Wi < 1 || Ho < 1 || Wo < 1 || KC < 8 || NC < 8 || R < 1 || S < 1) return -2;
  if ((KC % 8) || (NC % 8) || ((uintptr_t)in % 16) || ((uintptr_t)w % 16) || ((uintptr_t)out % 16)) return -3;
  if (res && ((uintptr_t)res % 16)) return -3;
  ConvGeom g;
  g.N = N; g.Ho = Ho; g.Wo = Wo; g.NC = NC; g.KC = KC; g.R = R; g.S = S;
  g.off_h = off_h; g.step_h = step_h; g.off_w = off_w; g.step_w = step_w;
  g.str_h = str_h; g.str_w = str_w;
  choose_box(Wo, Ho, N, CBM, &g.bw, &g.bh, &g.bnb);
  g.tiles_w = (Wo + g.bw - 1) / g.bw;
  g.tiles_h = (Ho + g.bh - 1) / g.bh;
  g.tiles_nb = (N + g.bnb - 1) / g.bnb;
  g.ldy = NC; g.b_mn = b_mn; g.act = act; g.bf16 = dtype == kBF16;
  g.log_bw = 0; g.log_bh = 0;
  while ((1 << g.log_bw) < g.bw) ++g.log_bw;
  while ((1 << g.log_bh) < g.bh) ++g.log_bh;
  g.fd_tiles_m = make_fastdiv((uint32_t)(g.tiles_w * g.tiles_h * g.tiles_nb));
  g.fd_tiles_w = make_fastdiv((uint32_t)g.tiles_w);
  g.fd_tiles_h = make_fastdiv((uint32_t)g.tiles_h);
  const long tiles_m = (long)g.tiles_w * g.tiles_h * g.tiles_nb;
  if (tiles_m * ((NC + 63) / 64) > 0x7fffffffL) return -2;
  const int bn = conv_pick_bn(tiles_m, NC);
  CUtensorMap mx, mw, my;
  int rc = make_map_nhwc(&mx, in, g.bf16, N, Hi, Wi, KC, g.bw, g.bh, g.bnb, in_sh, in_sw, str_h, str_w);
  if (rc) return rc;
  rc = make_map_filter(&mw, w, g.bf16, w_cout, R * S, w_cin, b_mn ? 64 : bn);
  if (rc) return rc;
  // every epilogue warp stores its 32 accumulator rows: a (sw x sh x sn) sub-box of the tile's pixel box
  const int sw = g.bw < 32 ? g.bw : 32;
  const int sh = g.bh < 32 / sw ? g.bh : 32 / sw;
  const int sn = 32 / (sw * sh);
  // with an output stride the stored tensor (out_full_h x out_full_w) is larger than the (Ho, Wo) pixel space of the tiles
  rc = make_map_store(&my, out, g.bf16, N, out_full_h > 0 ? out_full_h : Ho, out_full_w > 0 ? out_full_w : Wo, NC, sw, sh, sn,
                      out_sh, out_sw);
  if (rc) return rc;
#define MXB_CONV(T)                                                                              \
  (bn == 256 ? launch_conv<T, 256>(mx, mw, my, bias, res, stats, g, error_flag, st)               \
   : bn == 128 ? launch_conv<T, 128>(mx, mw, my, bias, res, stats, g, error_flag, st)             \
               : launch_conv<T, 64>(mx, mw, my, bias, res, stats, g, error_flag, st))
  return g.bf16 ? MXB_CONV(__nv_bfloat16) : MXB_CONV(__half);
#undef MXB_CONV
}

}  // namespace mxb

using namespace mxb;

// Cycle accounting of CTA 0 for the forward / data-gradient kernel: `buf` (16 int64 on the device, or null to switch it
// off) receives [0] producer cycles waiting for a free stage, [1] producer total, [2] k-steps issued, [3] MMA cycles
// waiting for operands, [4] MMA cycles waiting for a drained accumulator, [5] MMA total, [6] tiles, [7] first
// epilogue warp cycles waiting for an accumulator, [8] its total, [9] producer cycles in expect_tx, [10] in the TMA
// instruction, [11] MMA cycles in the four tcgen05.mma, [12] in tcgen05.commit, [13] / [14] remaining loop cycles of the
// producer / MMA warp.
MXB_EXPORT void mxb_conv_set_profile(long long* buf) { g_conv_prof = buf; }

// Rows of the statistics buffer written by mxb_conv_forward: [rows][2][Cout] floats (sum, sum of squares).
MXB_EXPORT int mxb_conv_stat_rows() { return sm_count() * 4; }

// y[N, Ho, Wo, Cout] = act(conv(x[N, H, W, Cin], w[Cout, R, S, Cin]) + bias + res), stride 1, Ho = H + 2*pad_h -
// dil_h*(R-1), Wo likewise.  Cin and Cout multiples of 8; pointers 16-byte aligned.  `stats` (optional):
// mxb_conv_stat_rows() * 2 * Cout floats, receives per-channel partial sums of y and y*y taken from the fp32 results.
MXB_EXPORT int mxb_conv_forward(int dtype, const void* x, const void* w, void* y, const void* bias, const void* res,
                                float* stats, int N, int H, int W, int Cin, int Cout, int R, int S, int pad_h, int pad_w,
                                int dil_h, int dil_w, int act, int* error_flag, void* stream) {
  const int Ho = H + 2 * pad_h - dil_h * (R - 1), Wo = W + 2 * pad_w - dil_w * (S - 1);
  return conv_run(dtype, x, w, y, bias, res, stats, N, H, W, Cin, Ho, Wo, Cout, R, S, -pad_h, dil_h, -pad_w, dil_w, Cout, Cin,
                  0, act, error_flag, (cudaStream_t)stream);
}

// Strided convolution with any filter size: Ho = (H + 2*pad_h - dil_h*(R-1) - 1) / sh + 1, Wo likewise.  The input boxes are
// fetched with traversal strides (sh, sw), so the contraction is the same loop over (tap, channel chunk).
MXB_EXPORT int mxb_conv_strided_forward(int dtype, const void* x, const void* w, void* y, const void* bias, float* stats, int N,
                                        int H, int W, int Cin, int Cout, int R, int S, int pad_h, int pad_w, int dil_h, int dil_w,
                                        int sh, int sw, int act, int* error_flag, void* stream) {
  if (sh < 1 || sw < 1) return -2;
  const int eh = H + 2 * pad_h - dil_h * (R - 1), ew = W + 2 * pad_w - dil_w * (S - 1);
  if (eh < 1 || ew < 1) return -2;
  const int Ho = (eh - 1) / sh + 1, Wo = (ew - 1) / sw + 1;
  return conv_run(dtype, x, w, y, bias, nullptr, stats, N, H, W, Cin, Ho, Wo, Cout, R, S, -pad_h, dil_h, -pad_w, dil_w, Cout, Cin, 0,
                  act, error_flag, (cudaStream_t)stream, 1, 1, 1, 1, 0, 0, sh, sw);
}

// Strided 1x1 convolution (the down-sampling shortcut of a residual network): y[N, Ho, Wo, Cout] with Ho = ceil(H / sh),
// Wo = ceil(W / sw) reads every sh-th row and sw-th column of x through a strided tensor map; same kernel.
MXB_EXPORT int mxb_conv1x1_strided_forward(int dtype, const void* x, const void* w, void* y, const void* bias, float* stats,
                                           int N, int H, int W, int Cin, int Cout, int sh, int sw, int act, int* error_flag,
                                           void* stream) {
  if (sh < 1 || sw < 1) return -2;
  const int Ho = (H + sh - 1) / sh, Wo = (W + sw - 1) / sw;
  return conv_run(dtype, x, w, y, bias, nullptr, stats, N, H, W, Cin, Ho, Wo, Cout, 1, 1, 0, 1, 0, 1, Cout, Cin, 0, act, error_flag,
                  (cudaStream_t)stream, sh, sw);
}

// Its data gradient: dx[N, H, W, Cin] is zero except at the sampled positions, which receive dy . w.  dx is cleared
// first, then the tiles are stored through a strided tensor map.
MXB_EXPORT int mxb_conv1x1_strided_dgrad(int dtype, const void* dy, const void* w, void* dx, int N, int H, int W, int Cin,
                                         int Cout, int sh, int sw, int* error_flag, void* stream) {
  if (sh < 1 || sw < 1) return -2;
  const int Ho = (H + sh - 1) / sh, Wo = (W + sw - 1) / sw;
  cudaError_t rc = cudaMemsetAsync(dx, 0, (size_t)N * H * W * Cin * 2, (cudaStream_t)stream);
  if (rc != cudaSuccess) return (int)rc;
  return conv_run(dtype, dy, w, dx, nullptr, nullptr, nullptr, N, Ho, Wo, Cout, Ho, Wo, Cin, 1, 1, 0, -1, 0, -1, Cout, Cin, 1, 0,
                  error_flag, (cudaStream_t)stream, 1, 1, sh, sw, H, W);
}

// dx[N, H, W, Cin] = sum_{r,s,co} dy[n, h + pad_h - r*dil_h, w + pad_w - s*dil_w, co] * w[co, r, s, Cin] (+ res):
// the data gradient of the stride-1 convolution above.  dy is [N, Ho, Wo, Cout].
MXB_EXPORT int mxb_conv_dgrad(int dtype, const void* dy, const void* w, void* dx, const void* res, int N, int H, int W,
                              int Cin, int Cout, int R, int S, int pad_h, int pad_w, int dil_h, int dil_w, int* error_flag,
                              void* stream) {
  const int Ho = H + 2 * pad_h - dil_h * (R - 1), Wo = W + 2 * pad_w - dil_w * (S - 1);
  return conv_run(dtype, dy, w, dx, nullptr, res, nullptr, N, Ho, Wo, Cout, H, W, Cin, R, S, pad_h, -dil_h, pad_w, -dil_w, Cout,
                  Cin, 1, 0, error_flag, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------------------------------
// Weight gradient:  dW[co, r, s, c] = sum_{n, h, w} dY[n, h, w, co] * X[n, h + off_h + r*step_h, w + off_w + s*step_w, c]
//
// Reference behaviour: cuDNN wgrad (src/operator/nn/cudnn/cudnn_convolution-inl.h) or im2col + GEMM.  Here it is a
// GEMM with M = Cout, N = Cin and the pixel axis as K; both operands are MN-major (channels contiguous), loaded as
// 4-D boxes of 64 pixels x 64 channels, the X box shifted by the tap offset with zero fill outside the image.  The
// pixel axis is split over CTAs (work unit = k-range x tap x output tile, taps innermost so that the CTAs running
// together read the same pixels through L2); each unit adds its fp32 tile into a zeroed fp32 buffer with vector
// reductions, and a small kernel converts the buffer to the weight's type.
// ------------------------------------------------------------------------------------------------------------------
namespace mxb {

struct WgradGeom {
  int N, Ho, Wo;                 // pixel space of dY
  int Cout, Cin, R, S;
  int off_h, step_h, off_w, step_w;
  int str_h, str_w;              // convolution stride: the x box of a k-step starts at (w0 * str_w + dw, h0 * str_h + dh)
  int kw, kh, knb;               // pixel box of one k-step, kw * kh * knb = 64
  int tiles_w, tiles_h, tiles_nb;
  int ksteps_per, ksplit;
  int bf16;
};

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename T, int BN>
__global__ void __launch_bounds__(kConvThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x,
                  float* __restrict__ dW32, const WgradGeom g, int* __restrict__ error_flag) {
  using Cfg = ConvCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr uint32_t B_BYTES = Cfg::B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * CA_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (CA_BYTES + B_BYTES) + Cfg::STAT_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + kConvMaxStages;
  uint64_t* acc_full = bars + 2 * kConvMaxStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_it = abort_flag + 1;
  volatile int* consumed_it = abort_flag + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = g.R * g.S;
  const int tiles_m = (g.Cout + CBM - 1) / CBM, tiles_n = (g.Cin + BN - 1) / BN;
  const int per_k = taps * tiles_m * tiles_n;
  const int num_units = per_k * g.ksplit;
  const int total_k = g.tiles_w * g.tiles_h * g.tiles_nb;
  constexpr uint32_t kTmemCols = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    *issued_it = 0;
    *consumed_it = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0, st = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok && !*abort_flag; u += gridDim.x) {
        const int ks = u / per_k, rest = u % per_k;
        const int tap = rest % taps, tm = (rest / taps) % tiles_m, tn = rest / (taps * tiles_m);
        const int r = tap / g.S, s = tap % g.S;
        const int dh = g.off_h + r * g.step_h, dw = g.off_w + s * g.step_w;
        const int k0 = ks * g.ksteps_per, k1 = min(total_k, k0 + g.ksteps_per);
        // pixel-box position of k-step k0, then advanced incrementally (w fastest, then h, then image group)
        int iw = k0 % g.tiles_w, ih = (k0 / g.tiles_w) % g.tiles_h, in = k0 / (g.tiles_w * g.tiles_h);
        for (int kt = k0; kt < k1; ++kt) {
          const int w0 = iw * g.kw, h0 = ih * g.kh, n0 = in * g.knb;
          if (!mbar_wait(&empty[st], ph ^ 1u)) { *abort_flag = 1; ok = false; break; }
          mbar_expect_tx(&full[st], CA_BYTES + B_BYTES);
#pragma unroll
          for (int c = 0; c < CBM / 64; ++c)
            tma_load_4d(sA + st * CA_BYTES + c * kMnChunkBytes, &map_dy, tm * CBM + c * 64, w0, h0, n0, &full[st]);
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            tma_load_4d(sB + st * B_BYTES + c * kMnChunkBytes, &map_x, tn * BN + c * 64, w0 * g.str_w + dw, h0 * g.str_h + dh, n0,
                        &full[st]);
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
          if (++iw == g.tiles_w) {
            iw = 0;
            if (++ih == g.tiles_h) { ih = 0; ++in; }
          }
        }
      }
      *issued_it = it;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(g.bf16, BN, 1, 1);
      constexpr uint64_t kstep = (16 * 128) >> 4;
      const uint64_t adesc0 = make_desc_mn(smem_u32(sA)), bdesc0 = make_desc_mn(smem_u32(sB));
      int it = 0, st = 0, t = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok && !*abort_flag; u += gridDim.x, ++t) {
        const int ks = u / per_k;
        const int k0 = ks * g.ksteps_per, k1 = min(total_k, k0 + g.ksteps_per);
        const int buf = t & 1;
        if (!mbar_wait(&acc_empty[buf], (((uint32_t)t >> 1) & 1u) ^ 1u)) { *abort_flag = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kt = k0; kt < k1; ++kt) {
          if (!mbar_wait(&full[st], ph)) { *abort_flag = 1; ok = false; break; }
          const uint64_t adesc = adesc0 + (uint64_t)(st * (int)(CA_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(st * (int)(B_BYTES >> 4));
          umma(tmem_d, adesc, bdesc, idesc, kt > k0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < CBK / CUMMA_K; ++k)
            umma(tmem_d, adesc + kstep * (uint64_t)k, bdesc + kstep * (uint64_t)k, idesc, 1u);
          umma_commit(&empty[st]);
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);
      }
      *consumed_it = it;
    }
  } else {
    const int q = warp & 3;
    int t = 0;
    for (int u = blockIdx.x; u < num_units; u += gridDim.x, ++t) {
      const int rest = u % per_k;
      const int tap = rest % taps, tm = (rest / taps) % tiles_m, tn = rest / (taps * tiles_m);
      const int buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], ((uint32_t)t >> 1) & 1u);
      if (!ready) *abort_flag = 1;
      if (!ready || *abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int co = tm * CBM + q * 32 + lane;
      const bool vec = (g.Cin % 4) == 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col0 = tn * BN + c0;
        uint32_t rr[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c0), rr);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (co < g.Cout && col0 < g.Cin) {
          float* drow = dW32 + ((size_t)co * taps + tap) * g.Cin + col0;
          if (vec && col0 + 32 <= g.Cin) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              red_add_v4(drow + v * 4, __uint_as_float(rr[v * 4]), __uint_as_float(rr[v * 4 + 1]), __uint_as_float(rr[v * 4 + 2]),
                         __uint_as_float(rr[v * 4 + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < g.Cin) atomicAdd(drow + j, __uint_as_float(rr[j]));
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    for (int it = *consumed_it; it < *issued_it; ++it) mbar_wait(&full[it % STAGES], (uint32_t)(it / STAGES) & 1u);
    if (error_flag) atomicExch(error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <typename T>
__global__ void __launch_bounds__(256) cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = Cvt<T>::from_f(src[i]);
}

template <typename T, int BN>
static int launch_wgrad(const CUtensorMap& mdy, const CUtensorMap& mx, float* dW32, void* dW, const WgradGeom& g, int* error_flag,
                        cudaStream_t st) {
  using Cfg = ConvCfg<BN>;
  static unsigned long long attr_seen = 0;
  if (first_on_device(&attr_seen)) {
    cudaError_t rc = cudaFuncSetAttribute(conv_wgrad_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (rc != cudaSuccess) return (int)rc;
  }
  const int64_t nw = (int64_t)g.Cout * g.R * g.S * g.Cin;
  cudaError_t rc = cudaMemsetAsync(dW32, 0, (size_t)nw * sizeof(float), st);
  if (rc != cudaSuccess) return (int)rc;
  const long units = (long)g.R * g.S * ((g.Cout + CBM - 1) / CBM) * ((g.Cin + BN - 1) / BN) * g.ksplit;
  const int grid = units < sm_count() ? (int)units : sm_count();
  conv_wgrad_kernel<T, BN><<<grid, kConvThreads, Cfg::SMEM_BYTES, st>>>(mdy, mx, dW32, g, error_flag);
  if (dW != nullptr) {
    const int cgrid = (int)((nw + 255) / 256 < 1184 ? (nw + 255) / 256 : 1184);
    cast_from_f32_kernel<T><<<cgrid, 256, 0, st>>>(dW32, (T*)dW, nw);
  }
  return (int)cudaGetLastError();
}

}  // namespace mxb

// dw[Cout, R, S, Cin] (type `dtype`; may be null to keep only the fp32 result) and dw32 (fp32 workspace of the same
// element count, overwritten) from x[N, H, W, Cin] and dy[N, Ho, Wo, Cout] of the stride-1 convolution above.
static int wgrad_run(int dtype, const void* x, const void* dy, void* dw, float* dw32, int N, int H, int W, int Cin, int Cout,
                     int R, int S, int pad_h, int pad_w, int dil_h, int dil_w, int sh, int sw, int* error_flag, void* stream,
                     int str_h = 1, int str_w = 1) {
  if (dtype != kF16 && dtype != kBF16) return -1;
  if (N < 1 || H < 1 || W < 1 || Cin < 8 || Cout < 8 || R < 1 || S < 1 || !dw32) return -2;
  if ((Cin % 8) || (Cout % 8) || ((uintptr_t)x % 16) || ((uintptr_t)dy % 16) || ((uintptr_t)dw32 % 16)) return -3;
  WgradGeom g;
  g.N = N; g.Ho = H + 2 * pad_h - dil_h * (R - 1); g.Wo = W + 2 * pad_w - dil_w * (S - 1);
  if (sh > 1 || sw > 1) { g.Ho = (H + sh - 1) / sh; g.Wo = (W + sw - 1) / sw; }      // strided 1x1: a sampled view of x
  if (g.Ho < 1 || g.Wo < 1) return -2;
  if (str_h > 1 || str_w > 1) { g.Ho = (g.Ho - 1) / str_h + 1; g.Wo = (g.Wo - 1) / str_w + 1; }      // strided R x S filter
  g.str_h = str_h; g.str_w = str_w;
  g.Cout = Cout; g.Cin = Cin; g.R = R; g.S = S;
  g.off_h = -pad_h; g.step_h = dil_h; g.off_w = -pad_w; g.step_w = dil_w;
  choose_box(g.Wo, g.Ho, N, 64, &g.kw, &g.kh, &g.knb);
  g.tiles_w = (g.Wo + g.kw - 1) / g.kw;
  g.tiles_h = (g.Ho + g.kh - 1) / g.kh;
  g.tiles_nb = (N + g.knb - 1) / g.knb;
  g.bf16 = dtype == kBF16;
  const int bn = Cin <= 64 ? 64 : (Cin <= 128 ? 128 : 256);
  const long per_k = (long)R * S * ((Cout + CBM - 1) / CBM) * ((Cin + bn - 1) / bn);
  const long total_k = (long)g.tiles_w * g.tiles_h * g.tiles_nb;
  if (total_k > 0x7fffffffL || per_k > 0x3fffffL) return -2;
  long ksplit = (4L * sm_count() + per_k - 1) / per_k;
  if (ksplit > total_k / 8) ksplit = total_k / 8;
  if (ksplit < 1) ksplit = 1;
  g.ksteps_per = (int)((total_k + ksplit - 1) / ksplit);
  g.ksplit = (int)((total_k + g.ksteps_per - 1) / g.ksteps_per);
  CUtensorMap mdy, mx;
  int rc = make_map_nhwc(&mdy, dy, g.bf16, N, g.Ho, g.Wo, Cout, g.kw, g.kh, g.knb);
  if (rc) return rc;
  rc = make_map_nhwc(&mx, x, g.bf16, N, H, W, Cin, g.kw, g.kh, g.knb, sh, sw, str_h, str_w);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
#define MXB_WGRAD(T)                                                                      \
  (bn == 256 ? launch_wgrad<T, 256>(mdy, mx, dw32, dw, g, error_flag, st)                  \
   : bn == 128 ? launch_wgrad<T, 128>(mdy, mx, dw32, dw, g, error_flag, st)                \
               : launch_wgrad<T, 64>(mdy, mx, dw32, dw, g, error_flag, st))
  return g.bf16 ? MXB_WGRAD(__nv_bfloat16) : MXB_WGRAD(__half);
#undef MXB_WGRAD
}

MXB_EXPORT int mxb_conv_wgrad(int dtype, const void* x, const void* dy, void* dw, float* dw32, int N, int H, int W, int Cin,
                              int Cout, int R, int S, int pad_h, int pad_w, int dil_h, int dil_w, int* error_flag,
                              void* stream) {
  return wgrad_run(dtype, x, dy, dw, dw32, N, H, W, Cin, Cout, R, S, pad_h, pad_w, dil_h, dil_w, 1, 1, error_flag, stream);
}

// Weight gradient of the strided convolution with any filter size: dy is [N, Ho, Wo, Cout] with Ho, Wo as in
// mxb_conv_strided_forward.
MXB_EXPORT int mxb_conv_strided_wgrad(int dtype, const void* x, const void* dy, void* dw, float* dw32, int N, int H, int W, int Cin,
                                      int Cout, int R, int S, int pad_h, int pad_w, int dil_h, int dil_w, int sh, int sw,
                                      int* error_flag, void* stream) {
  if (sh < 1 || sw < 1) return -2;
  return wgrad_run(dtype, x, dy, dw, dw32, N, H, W, Cin, Cout, R, S, pad_h, pad_w, dil_h, dil_w, 1, 1, error_flag, stream, sh, sw);
}

// Weight gradient of the strided 1x1 convolution: dy is [N, ceil(H / sh), ceil(W / sw), Cout].
MXB_EXPORT int mxb_conv1x1_strided_wgrad(int dtype, const void* x, const void* dy, void* dw, float* dw32, int N, int H, int W,
                                         int Cin, int Cout, int sh, int sw, int* error_flag, void* stream) {
  if (sh < 1 || sw < 1) return -2;
  return wgrad_run(dtype, x, dy, dw, dw32, N, H, W, Cin, Cout, 1, 1, 0, 0, 1, 1, sh, sw, error_flag, stream);
}

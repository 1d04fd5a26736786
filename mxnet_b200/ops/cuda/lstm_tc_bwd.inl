// Backward recurrence of lstm_tc.cu (included inside namespace mxb).
//
// The gate gradients of step t are written once, as rows t*B .. t*B+B of `dgates` [T*B, KK], and that is also what the
// product of the step streams: its box of Bp >= B rows runs into the rows of step t+1 (written in an earlier phase; they
// only reach accumulator lanes that nobody reads) or, for the last step, past the end of the tensor (zero fill).
// Dynamic shared memory: [ring: stages x Bp x 128][Wb: KK/KC chunks x UB x 128][slack][TcShared], UB = max(U, 8) rows per
// chunk.  The MMA has N = 16 columns; with U = 8 its second group of eight rows is whatever follows the chunk and lands in
// accumulator columns 8..15, which nobody reads.
template <typename T, typename X, int U>
__global__ void __launch_bounds__(kTcThreads, 1)
lstm_tc_bwd_kernel(const __grid_constant__ CUtensorMap map_dg, const __grid_constant__ CUtensorMap map_wb, const LstmTcParams p) {
  constexpr int KC = TcType<X>::KC;
  constexpr int NG = 4 * U;
  constexpr uint32_t WB_CHUNK = U * 128;
  constexpr uint32_t TMEM_COLS = 32;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int nk = p.KK / KC;
  const uint32_t stage_bytes = (uint32_t)p.Bp * 128u;
  uint8_t* ring = smem;
  uint8_t* sW = ring + (size_t)p.stages * stage_bytes;
  TcShared* sh = reinterpret_cast<TcShared*>(sW + (size_t)nk * WB_CHUNK + 2048);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const unsigned int nctas = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    mbar_init(&sh->acc_full, 1);
    mbar_init(&sh->w_full, 1);
    sh->abort_flag = 0;
    sh->issued_it = 0;
    sh->consumed_it = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh->tmem_slot;

  __shared__ int step_ok;
  if (threadIdx.x == 0) {
    mbar_expect_tx(&sh->w_full, (uint32_t)nk * WB_CHUNK);
    for (int kc = 0; kc < nk; ++kc) tma_load_2d(sW + (size_t)kc * WB_CHUNK, &map_wb, kc * KC, cta * U, &sh->w_full);
    const bool ok = tc_mbar_wait(&sh->w_full, 0);
    if (!ok) { sh->abort_flag = 1; tc_fail(p.bar, 5u); }
    step_ok = ok ? 1 : 0;
  }
  __syncthreads();
  bool alive = step_ok != 0;

  const int q = warp & 3;
  const int b = q * 32 + lane;
  const bool epi = warp >= 2;
  const bool row_ok = epi && b < p.B;
  const int unit0 = cta * U;
  float dc[U];                                   // carried cell gradient of this thread's (batch row, units)
#pragma unroll
  for (int u = 0; u < U; ++u)
    dc[u] = (row_ok && p.dcT && unit0 + u < p.H) ? Cvt<T>::to_f(static_cast<const T*>(p.dcT)[(size_t)b * p.H + unit0 + u]) : 0.f;

  int pst = 0, pit = 0, cst = 0, cit = 0;
  uint32_t pph = 0, cph = 0;
  const uint32_t idesc = tc_idesc(TcType<X>::FMT, 16);
  // phase s: the epilogue turns (dy_t, recurrent dh from product s-1, carried dc) into the gate gradients of step
  // t = T-1-s; after the barrier the product of phase s contracts them with W_hh.  Phase T only collects dh0 / dc0.
  for (int s = 0; s <= p.T && alive; ++s) {
    const int t = p.T - 1 - s;
    if (epi) {
      float rec[U];
      bool ready = true;
      if (s > 0) {
        ready = tc_mbar_wait_warp(&sh->acc_full, (uint32_t)(s - 1) & 1u);
        if (!ready) { sh->abort_flag = 1; tc_fail(p.bar, 4u); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ready) {                              // warp-wide: tcgen05.ld is .sync.aligned
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16), r);
          tmem_wait_ld32(r);
#pragma unroll
          for (int u = 0; u < U; ++u) rec[u] = __uint_as_float(r[u]);
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u)
          rec[u] = (row_ok && p.dhT && unit0 + u < p.H) ? Cvt<T>::to_f(static_cast<const T*>(p.dhT)[(size_t)b * p.H + unit0 + u]) : 0.f;
      }
      if (ready && row_ok) {
        if (s == p.T) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (unit0 + u < p.H) {
              static_cast<T*>(p.dh0)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(rec[u]);
              static_cast<T*>(p.dc0)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(dc[u]);
            }
        } else {
          const int nvalid = p.H - unit0 < U ? p.H - unit0 : U;
          float gt[NG], ctv[U], cpv[U], dyv[U];
          tc_ld_w<T, NG, 16>(static_cast<const T*>(p.gates) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NG, gt);
          tc_ld_w<float, U, 16>(p.cs + ((size_t)t * p.B + b) * p.Hc + unit0, ctv);
          if (t > 0) tc_ld_w<float, U, 16>(p.cs + ((size_t)(t - 1) * p.B + b) * p.Hc + unit0, cpv);
          else tc_ld_row<T, U>(static_cast<const T*>(p.c0) + (size_t)b * p.H + unit0, cpv, 0, nvalid);
          tc_ld_row<T, U>(static_cast<const T*>(p.dy) + ((size_t)t * p.B + b) * p.H + unit0, dyv, p.yalign, nvalid);
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const bool ok = unit0 + u < p.H;
            const float ig = gt[u], fg = gt[U + u], gg = gt[2 * U + u], og = gt[3 * U + u];
            const float dh = rec[u] + dyv[u];
            const float th = tc_tanh(ctv[u]);
            const float dct = dc[u] + dh * og * (1.f - th * th);
            dc[u] = dct * fg;
            gt[u] = ok ? dct * gg * ig * (1.f - ig) : 0.f;
            gt[U + u] = ok ? dct * cpv[u] * fg * (1.f - fg) : 0.f;
            gt[2 * U + u] = ok ? dct * ig * (1.f - gg * gg) : 0.f;
            gt[3 * U + u] = ok ? dh * th * og * (1.f - og) : 0.f;
          }
          tc_st_w<T, NG, 16>(static_cast<T*>(p.dgates) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NG, gt);
          tc_fence_async_global();
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (s == p.T) break;
    __syncthreads();
    if (threadIdx.x == 0) {
      bool ok = sh->abort_flag == 0;
      if (!ok) tc_fail(p.bar, 6u);
      if (ok) ok = tc_grid_arrive_wait(p.bar, (unsigned int)(s + 1) * nctas);
      tc_fence_async_global();
      step_ok = ok ? 1 : 0;
    }
    __syncthreads();
    alive = step_ok != 0;
    if (!alive) break;
    if (warp == 0) {
      if (lane == 0) {
        tc_produce<X>(sh, p.bar, ring, stage_bytes, p.stages, &map_dg, t * p.B, nk, pst, pph, pit);
        sh->issued_it = pit;
      }
    } else if (warp == 1) {
      if (lane == 0) {
        tc_consume<X>(sh, p.bar, ring, stage_bytes, p.stages, sW, WB_CHUNK, nk, tmem_base, idesc, cst, cph, cit);
        sh->consumed_it = cit;
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && sh->abort_flag) {
    for (int it = sh->consumed_it; it < sh->issued_it; ++it) tc_mbar_wait(&sh->full[it % p.stages], (uint32_t)(it / p.stages) & 1u);
    tc_fail(p.bar, 6u);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

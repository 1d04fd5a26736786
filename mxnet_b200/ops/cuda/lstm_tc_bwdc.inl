// Backward recurrence of lstm_tc.cu with the contraction axis cut over a cluster of four CTAs (included inside
// namespace mxb).
//
// In lstm_tc_bwd_kernel every CTA streams the whole gate-gradient matrix of the step from L2, which bounds a step by the
// L2-to-SM rate.  Here the four CTAs of a cluster together own 4U hidden units: CTA r of the cluster keeps the columns
// [r * KK/4, (r+1) * KK/4) of W_hh for all 4U units in shared memory, streams only that quarter of the gate gradients, and
// gets partial sums for all 4U units in TMEM.  The CTAs then hand each other the partial sums of the units the receiver
// owns through distributed shared memory (one 16- or 32-byte row per batch row and sender), meet at a cluster barrier,
// and each adds the four parts for its own U units.  Everything else (ownership of the cell update, layouts, grid barrier,
// bounded waits) is as in lstm_tc_bwd_kernel.  The cluster barrier is a hardware barrier: every CTA executes it in every
// phase, also after a failed wait; before it each CTA tells its partners whether its last grid barrier succeeded, and the
// four leave the loop together when any of them failed (a CTA that left alone would hang the others at the next cluster
// barrier).
//
// Dynamic shared memory: [ring: stages x Bp x 128][Wb: (KK/4)/KC chunks x 4U x 128][xbuf: 4 x 128 x U floats][xflag: 4][TcShared].
constexpr int kTcCluster = 4;

__device__ __forceinline__ void st_cluster_f4(uint32_t cluster_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename T, typename X, int U>
__global__ void __launch_bounds__(kTcThreads, 1)
lstm_tc_bwdc_kernel(const __grid_constant__ CUtensorMap map_dg, const __grid_constant__ CUtensorMap map_wb, const LstmTcParams p) {
  constexpr int KC = TcType<X>::KC;
  constexpr int NG = 4 * U;
  constexpr int UC = kTcCluster * U;                       // units of the cluster = columns of the MMA
  constexpr uint32_t WB_CHUNK = UC * 128;
  constexpr uint32_t TMEM_COLS = UC < 32 ? 32 : UC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int kks = p.KK / kTcCluster;                       // contraction columns of this CTA
  const int nk = kks / KC;
  const uint32_t stage_bytes = (uint32_t)p.Bp * 128u;
  uint8_t* ring = smem;
  uint8_t* sW = ring + (size_t)p.stages * stage_bytes;
  float* xbuf = reinterpret_cast<float*>(sW + (size_t)nk * WB_CHUNK);           // [sender][batch row][U]
  volatile int* xflag = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(xbuf) + (size_t)kTcCluster * 128 * U * sizeof(float));
  TcShared* sh = reinterpret_cast<TcShared*>(const_cast<int*>(xflag) + 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int crank = (int)cluster_ctarank();
  const int cluster_id = cta / kTcCluster;
  const unsigned int nctas = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    mbar_init(&sh->acc_full, 1);
    mbar_init(&sh->w_full, 1);
    sh->abort_flag = 0;
    sh->issued_it = 0;
    sh->consumed_it = 0;
    for (int d = 0; d < kTcCluster; ++d) xflag[d] = 1;
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
    for (int kc = 0; kc < nk; ++kc)
      tma_load_2d(sW + (size_t)kc * WB_CHUNK, &map_wb, crank * kks + kc * KC, cluster_id * UC, &sh->w_full);
    const bool ok = tc_mbar_wait(&sh->w_full, 0);
    if (!ok) { sh->abort_flag = 1; tc_fail(p.bar, 5u); }
    step_ok = 1;                       // a failed load is reported at the first grid barrier, where every CTA leaves
  }
  __syncthreads();
  cluster_sync_all();                  // every CTA of the cluster is running before anyone writes into its shared memory
  bool alive = true;          // the cluster's verdict: all four CTAs passed their last grid barrier
  bool mine = true;           // this CTA's own

  const int q = warp & 3;
  const int b = q * 32 + lane;
  const bool epi = warp >= 2;
  const bool row_ok = epi && b < p.B;
  const int unit0 = cta * U;
  float dc[U];
#pragma unroll
  for (int u = 0; u < U; ++u)
    dc[u] = (row_ok && p.dcT && unit0 + u < p.H) ? Cvt<T>::to_f(static_cast<const T*>(p.dcT)[(size_t)b * p.H + unit0 + u]) : 0.f;

  int pst = 0, pit = 0, cst = 0, cit = 0;
  uint32_t pph = 0, cph = 0;
  const uint32_t idesc = tc_idesc(TcType<X>::FMT, UC);
  for (int s = 0; s <= p.T && alive; ++s) {
    const int t = p.T - 1 - s;
    float rec[U];
    bool ready = true;
    if (s > 0) {
      if (threadIdx.x == 0) {
        for (int d = 0; d < kTcCluster; ++d)
          asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(mapa_u32(smem_u32(const_cast<int*>(xflag) + crank), (uint32_t)d)), "r"(mine ? 1 : 0) : "memory");
      }
      if (epi) {
        ready = mine && tc_mbar_wait_warp(&sh->acc_full, (uint32_t)(s - 1) & 1u);
        if (mine && !ready) { sh->abort_flag = 1; tc_fail(p.bar, 4u); }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float v[UC];
        if (ready) tc_tmem_load<UC>(tmem_base + ((uint32_t)(q * 32) << 16), v);          // warp-wide
        if (ready && row_ok) {
#pragma unroll
          for (int d = 0; d < kTcCluster; ++d) {
            if (d == crank) {
#pragma unroll
              for (int u = 0; u < U; ++u) rec[u] = v[d * U + u];
            } else {
              // the partial sums of CTA d's units go into its exchange buffer, slot [this CTA][batch row]
              const uint32_t dst = mapa_u32(smem_u32(xbuf + ((size_t)crank * 128 + b) * U), (uint32_t)d);
#pragma unroll
              for (int u = 0; u < U; u += 4) st_cluster_f4(dst + (uint32_t)u * 4u, v[d * U + u], v[d * U + u + 1], v[d * U + u + 2], v[d * U + u + 3]);
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      }
      cluster_sync_all();              // all four partial sums have landed (release / acquire at cluster scope)
      alive = xflag[0] && xflag[1] && xflag[2] && xflag[3];
      if (!alive) break;
      if (epi && ready && row_ok) {
#pragma unroll
        for (int d = 0; d < kTcCluster; ++d)
          if (d != crank) {
            const float* src = xbuf + ((size_t)d * 128 + b) * U;
#pragma unroll
            for (int u = 0; u < U; u += 4) {
              const float4 x4 = *reinterpret_cast<const float4*>(src + u);
              rec[u] += x4.x; rec[u + 1] += x4.y; rec[u + 2] += x4.z; rec[u + 3] += x4.w;
            }
          }
      }
    } else {
#pragma unroll
      for (int u = 0; u < U; ++u)
        rec[u] = (row_ok && p.dhT && unit0 + u < p.H) ? Cvt<T>::to_f(static_cast<const T*>(p.dhT)[(size_t)b * p.H + unit0 + u]) : 0.f;
    }
    if (epi && ready && row_ok) {
      if (s == p.T) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (unit0 + u < p.H) {
            static_cast<T*>(p.dh0)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(rec[u]);
            static_cast<T*>(p.dc0)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(dc[u]);
          }
      } else {
        const int nvalid = p.H - unit0 < U ? (p.H - unit0 > 0 ? p.H - unit0 : 0) : U;
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
    mine = step_ok != 0;
    if (mine && warp == 0) {
      if (lane == 0) {
        // this CTA's quarter of the gate gradients: columns crank * kks ..., rows of step t
        for (int kc = 0; kc < nk; ++kc) {
          if (!tc_mbar_wait(&sh->empty[pst], pph ^ 1u)) { sh->abort_flag = 1; tc_fail(p.bar, 2u); break; }
          mbar_expect_tx(&sh->full[pst], stage_bytes);
          tma_load_2d(ring + (size_t)pst * stage_bytes, &map_dg, crank * kks + kc * KC, t * p.B, &sh->full[pst]);
          ++pit;
          if (++pst == p.stages) { pst = 0; pph ^= 1u; }
        }
        sh->issued_it = pit;
      }
    } else if (mine && warp == 1) {
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
  cluster_sync_all();                  // nobody leaves while a partner may still address its shared memory
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

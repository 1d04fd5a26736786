// GRU recurrence on the tensor cores (included by lstm_tc.cu inside namespace mxb; same building blocks as the LSTM kernels).
//
// Reference behaviour: the `RNN` operator in gru mode (src/operator/rnn-inl.h; CPU math in src/operator/rnn_impl.h,
// GruForwardTraining / GruBackward).  Gate order r, z, n:
//     r = sigmoid(xr + hr), z = sigmoid(xz + hz), n = tanh(xn + r * (hn + b_hn)), h_t = (1 - z) * n + z * h_{t-1}
// with x* = x_t W_ih^T + b_ih (+ b_hh for r and z) from the input GEMM and h* = h_{t-1} W_hh^T from the per-step product.
// A CTA owns U hidden units; its 3U gate rows are padded to NGP = one 128-byte chunk of elements (32 for fp32, 64 for half
// precision), so every per-thread row of the gate-major arrays is a whole number of 16-byte vectors and a quarter of the
// contraction axis of the backward pass is a whole number of chunks.  Thread b keeps h of its units in registers.
// Backward (clusters of four CTAs as lstm_tc_bwdc_kernel): the gradient with respect to h_{t-1} is dh * z (kept in
// registers) plus W_hh^T applied to the hidden-side gate gradients [dar, daz, dan * r], which are what the product
// streams; the input side needs [dar, daz, dan], written beside them for the GEMMs outside.

struct GruTcParams {
  LstmTcParams base;       // xproj [T, B, KK] (columns c*NGP + g*U + u), y, hT, gates [T, B, KK], hbuf, bar, T, B, H, Bp, Hp, Hc, KK,
                           // stages, yalign; backward: dy, dhT, dgates (= hidden-side gradients [T, B, KK]), dh0
  const void* bhn;         // [Hc] hidden-side bias of the candidate gate, fp32, zero padded
  float* hnb;              // [T, B, Hc] h_{t-1} W_hn + b_hn (saved for backward; may be null)
  void* dgx;               // [T, B, KK] input-side gate gradients (backward output)
  const void* h0;          // [B, H]
};

template <typename T, typename X, int U>
__global__ void __launch_bounds__(kTcThreads, 1)
gru_tc_fwd_kernel(const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_w, const GruTcParams gp) {
  const LstmTcParams& p = gp.base;
  constexpr int KC = TcType<X>::KC;
  constexpr int NGP = KC;                                  // padded gate columns of a CTA (3U real ones)
  static_assert(3 * U <= NGP, "three gates of U units fit one chunk");
  constexpr uint32_t W_CHUNK = NGP * 128;
  constexpr uint32_t TMEM_COLS = NGP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int nk = p.Hp / KC;
  const uint32_t stage_bytes = (uint32_t)p.Bp * 128u;
  uint8_t* ring = smem;
  uint8_t* sW = ring + (size_t)p.stages * stage_bytes;
  TcShared* sh = reinterpret_cast<TcShared*>(sW + (size_t)nk * W_CHUNK);
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

  if (threadIdx.x == 0) {
    mbar_expect_tx(&sh->w_full, (uint32_t)nk * W_CHUNK);
    for (int kc = 0; kc < nk; ++kc) tma_load_2d(sW + (size_t)kc * W_CHUNK, &map_w, kc * KC, cta * NGP, &sh->w_full);
  }

  const int q = warp & 3;
  const int b = q * 32 + lane;
  const bool epi = warp >= 2;
  const bool row_ok = epi && b < p.B;
  const int unit0 = cta * U;
  float hp[U], bh[U];                                      // h of this thread's units, and their candidate-gate bias
  X* hbuf = static_cast<X*>(p.hbuf);
#pragma unroll
  for (int u = 0; u < U; ++u) { hp[u] = 0.f; bh[u] = 0.f; }
  if (row_ok) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = unit0 + u < p.H;
      hp[u] = ok ? Cvt<T>::to_f(static_cast<const T*>(gp.h0)[(size_t)b * p.H + unit0 + u]) : 0.f;
      bh[u] = static_cast<const float*>(gp.bhn)[unit0 + u];
      if (ok) hbuf[(size_t)b * p.Hp + unit0 + u] = Cvt<X>::from_f(hp[u]);
    }
    tc_fence_async_global();
  }
  __syncthreads();
  __shared__ int step_ok;
  if (threadIdx.x == 0) {
    bool ok = tc_grid_arrive_wait(p.bar, nctas);
    if (ok && !tc_mbar_wait(&sh->w_full, 0)) { ok = false; tc_fail(p.bar, 5u); }
    tc_fence_async_global();
    step_ok = ok ? 1 : 0;
  }
  __syncthreads();
  bool alive = step_ok != 0;

  int pst = 0, pit = 0, cst = 0, cit = 0;
  uint32_t pph = 0, cph = 0;
  const uint32_t idesc = tc_idesc(TcType<X>::FMT, NGP);
  for (int t = 0; t < p.T && alive; ++t) {
    const int par = t & 1;
    if (warp == 0) {
      if (lane == 0) {
        tc_produce<X>(sh, p.bar, ring, stage_bytes, p.stages, &map_h, par * p.Bp, nk, pst, pph, pit);
        sh->issued_it = pit;
      }
    } else if (warp == 1) {
      if (lane == 0) {
        tc_consume<X>(sh, p.bar, ring, stage_bytes, p.stages, sW, W_CHUNK, nk, tmem_base, idesc, cst, cph, cit);
        sh->consumed_it = cit;
      }
    } else {
      float a[NGP];
      if (row_ok) tc_ld_w<T, NGP, 16>(static_cast<const T*>(p.xproj) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NGP, a);
      const bool ready = tc_mbar_wait_warp(&sh->acc_full, (uint32_t)t & 1u);
      if (!ready) { sh->abort_flag = 1; tc_fail(p.bar, 4u); }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float v[NGP];
      if (ready) tc_tmem_load<NGP>(tmem_base + ((uint32_t)(q * 32) << 16), v);      // warp-wide
      if (ready && row_ok) {
        float hnbv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float r = tc_sigmoid(a[u] + v[u]);
          const float z = tc_sigmoid(a[U + u] + v[U + u]);
          hnbv[u] = v[2 * U + u] + bh[u];
          const float n = tc_tanh(a[2 * U + u] + r * hnbv[u]);
          hp[u] = unit0 + u < p.H ? (1.f - z) * n + z * hp[u] : 0.f;
          a[u] = r;
          a[U + u] = z;
          a[2 * U + u] = n;
        }
        const int nvalid = p.H - unit0 < U ? (p.H - unit0 > 0 ? p.H - unit0 : 0) : U;
        tc_st_w<X, U, 16>(hbuf + ((size_t)(par ^ 1) * p.Bp + b) * p.Hp + unit0, hp);
        tc_st_row<T, U>(static_cast<T*>(p.y) + ((size_t)t * p.B + b) * p.H + unit0, hp, p.yalign, nvalid);
        if (p.gates) tc_st_w<T, NGP, 16>(static_cast<T*>(p.gates) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NGP, a);
        if (gp.hnb) tc_st_w<float, U, 16>(gp.hnb + ((size_t)t * p.B + b) * p.Hc + unit0, hnbv);
        if (t == p.T - 1) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (unit0 + u < p.H) static_cast<T*>(p.hT)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(hp[u]);
        }
        tc_fence_async_global();
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      bool ok = sh->abort_flag == 0;
      if (!ok) tc_fail(p.bar, 6u);
      if (ok && t + 1 < p.T) ok = tc_grid_arrive_wait(p.bar, (unsigned int)(t + 2) * nctas);
      tc_fence_async_global();
      step_ok = ok ? 1 : 0;
    }
    __syncthreads();
    alive = step_ok != 0;
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

// Backward, clusters of four CTAs (structure and exit protocol of lstm_tc_bwdc_kernel).
// Dynamic shared memory: [ring][Wb: (KK/4)/KC chunks x 4U x 128][xbuf: 4 x 128 x U floats][xflag][TcShared].
template <typename T, typename X, int U>
__global__ void __launch_bounds__(kTcThreads, 1)
gru_tc_bwdc_kernel(const __grid_constant__ CUtensorMap map_dg, const __grid_constant__ CUtensorMap map_wb, const GruTcParams gp) {
  const LstmTcParams& p = gp.base;
  constexpr int KC = TcType<X>::KC;
  constexpr int NGP = KC;
  constexpr int UC = kTcCluster * U;
  constexpr uint32_t WB_CHUNK = UC * 128;
  constexpr uint32_t TMEM_COLS = UC < 32 ? 32 : UC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int kks = p.KK / kTcCluster;
  const int nk = kks / KC;
  const uint32_t stage_bytes = (uint32_t)p.Bp * 128u;
  uint8_t* ring = smem;
  uint8_t* sW = ring + (size_t)p.stages * stage_bytes;
  float* xbuf = reinterpret_cast<float*>(sW + (size_t)nk * WB_CHUNK);
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
    step_ok = 1;
  }
  __syncthreads();
  cluster_sync_all();
  bool alive = true, mine = true;

  const int q = warp & 3;
  const int b = q * 32 + lane;
  const bool epi = warp >= 2;
  const bool row_ok = epi && b < p.B;
  const int unit0 = cta * U;
  float dhd[U];                                            // dh_t * z_t: the part of dh_{t-1} that does not go through W_hh
#pragma unroll
  for (int u = 0; u < U; ++u) dhd[u] = 0.f;

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
        if (ready) tc_tmem_load<UC>(tmem_base + ((uint32_t)(q * 32) << 16), v);
        if (ready && row_ok) {
#pragma unroll
          for (int d = 0; d < kTcCluster; ++d) {
            if (d == crank) {
#pragma unroll
              for (int u = 0; u < U; ++u) rec[u] = v[d * U + u];
            } else {
              const uint32_t dst = mapa_u32(smem_u32(xbuf + ((size_t)crank * 128 + b) * U), (uint32_t)d);
#pragma unroll
              for (int u = 0; u < U; u += 4) st_cluster_f4(dst + (uint32_t)u * 4u, v[d * U + u], v[d * U + u + 1], v[d * U + u + 2], v[d * U + u + 3]);
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      }
      cluster_sync_all();
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
#pragma unroll
        for (int u = 0; u < U; ++u) rec[u] += dhd[u];
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
          if (unit0 + u < p.H) static_cast<T*>(p.dh0)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(rec[u]);
      } else {
        const int nvalid = p.H - unit0 < U ? (p.H - unit0 > 0 ? p.H - unit0 : 0) : U;
        float gt[NGP], gx[NGP], hnbv[U], hpv[U], dyv[U];
        tc_ld_w<T, NGP, 16>(static_cast<const T*>(p.gates) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NGP, gt);
        tc_ld_w<float, U, 16>(gp.hnb + ((size_t)t * p.B + b) * p.Hc + unit0, hnbv);
        if (t > 0) tc_ld_row<T, U>(static_cast<const T*>(p.y) + ((size_t)(t - 1) * p.B + b) * p.H + unit0, hpv, p.yalign, nvalid);
        else tc_ld_row<T, U>(static_cast<const T*>(gp.h0) + (size_t)b * p.H + unit0, hpv, 0, nvalid);
        tc_ld_row<T, U>(static_cast<const T*>(p.dy) + ((size_t)t * p.B + b) * p.H + unit0, dyv, p.yalign, nvalid);
#pragma unroll
        for (int j = 3 * U; j < NGP; ++j) { gt[j] = 0.f; }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const bool ok = unit0 + u < p.H;
          const float r = gt[u], z = gt[U + u], n = gt[2 * U + u];
          const float dh = rec[u] + dyv[u];
          const float dn = dh * (1.f - z);
          const float dz = dh * (hpv[u] - n);
          dhd[u] = ok ? dh * z : 0.f;
          const float dan = dn * (1.f - n * n);
          const float dar = dan * hnbv[u] * r * (1.f - r);
          const float daz = dz * z * (1.f - z);
          gt[u] = ok ? dar : 0.f;
          gt[U + u] = ok ? daz : 0.f;
          gt[2 * U + u] = ok ? dan * r : 0.f;              // hidden side: through r * (hn + b_hn)
          gx[u] = gt[u];
          gx[U + u] = gt[U + u];
          gx[2 * U + u] = ok ? dan : 0.f;                  // input side
        }
#pragma unroll
        for (int j = 3 * U; j < NGP; ++j) gx[j] = 0.f;
        tc_st_w<T, NGP, 16>(static_cast<T*>(p.dgates) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NGP, gt);
        tc_st_w<T, NGP, 16>(static_cast<T*>(gp.dgx) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NGP, gx);
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
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

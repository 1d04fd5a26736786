// Fused self-attention for sequences longer than one 128-row tile (included by attention.cu inside namespace mxb).
//
// Forward: one CTA per (sample, head, block of 128 queries) walks the key/value blocks of 128 with the running
// maximum / sum of the streaming softmax.  Per key block the tensor cores produce S = Q Kt into TMEM, the row threads
// turn it into P (shared memory, operand layout) and the tensor cores produce the block's P V into a second TMEM
// region; the row threads fold that into an output row held in registers, rescaled when the maximum moves.  The K and V
// tiles are single buffers that are reloaded as soon as the product that read them has completed, so the loads run
// under the softmax of the same block.  Two CTAs fit one SM (shared memory, 256 TMEM columns each) and cover each
// other's serial phases.
//
// Backward: one CTA per (sample, head, block of 128 keys) keeps K and V of its block resident and walks the query
// blocks (Q and dO double buffered).  dK and dV accumulate in TMEM over the whole walk; the block's contribution to dQ
// is a fresh product per query block, written in fp32 to the slot of this key block; a short kernel adds the slots in
// a fixed order (deterministic) and writes dQ in the model's type.
// Every wait is bounded and warp-uniform where a warp-wide instruction follows.

constexpr int kAttLongMaxT = 1024;
constexpr uint32_t kFwdLongSmem = 5 * kTileBytes + kAttLongMaxT * 4 + 1024 + 256;

template <typename T>
__global__ void __launch_bounds__(kAttThreads, 2)
attn_fwd_long_kernel(const __grid_constant__ CUtensorMap map_qkv, const AttnParams p, int bf16) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  uint8_t* sP = smem + 3 * kTileBytes;                 // two k-stages of P: keys 0..63, 64..127 of the block
  float* kbias = reinterpret_cast<float*>(smem + 5 * kTileBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(kbias + kAttLongMaxT);
  uint64_t* bar_q = bars, *bar_k = bars + 1, *bar_v = bars + 2, *bar_s = bars + 3, *bar_p = bars + 4, *bar_o = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.T + kAttT - 1) / kAttT;
  const int qi = blockIdx.x % nblk;
  const int bh = blockIdx.x / nblk;
  const int b = bh / p.heads, h = bh % p.heads;
  constexpr uint32_t kTmemCols = 256;                  // S: columns [0, 128), block P V: [128, 192)

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 4); mbar_init(bar_o, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int k = threadIdx.x; k < nblk * kAttT; k += kAttThreads) {
    bool valid = k < p.T;
    if (valid && p.mask) valid = static_cast<const float*>(p.mask)[(int64_t)b * p.T + k] != 0.f;
    kbias[k] = valid ? 0.f : -INFINITY;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_q, kTileBytes);
      tma_load_3d(sQ, &map_qkv, h * kAttD, qi * kAttT, b, bar_q);
      for (int j = 0; j < nblk; ++j) {
        // the K tile is free once S of the previous block is complete, the V tile once its P V is
        if (j > 0 && !mbar_wait(bar_s, (uint32_t)(j - 1) & 1u)) { *abort_flag = 1; break; }
        mbar_expect_tx(bar_k, kTileBytes);
        tma_load_3d(sK, &map_qkv, p.C + h * kAttD, j * kAttT, b, bar_k);
        if (j > 0 && !mbar_wait(bar_o, (uint32_t)(j - 1) & 1u)) { *abort_flag = 1; break; }
        mbar_expect_tx(bar_v, kTileBytes);
        tma_load_3d(sV, &map_qkv, 2 * p.C + h * kAttD, j * kAttT, b, bar_v);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(bar_q, 0);
      const uint32_t idesc = make_idesc(bf16, 128, 0, 0);
      const uint32_t idesc2 = make_idesc(bf16, kAttD, 0, 1);             // A = P K-major, B = V MN-major, N = 64
      const uint64_t qd = make_desc(smem_u32(sQ)), kd = make_desc(smem_u32(sK));
      const uint32_t v_addr = smem_u32(sV);
      for (int j = 0; j < nblk && ok; ++j) {
        const uint32_t ph = (uint32_t)j & 1u;
        ok = mbar_wait(bar_k, ph);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k = 0; k < kAttD / 16; ++k) umma(tmem_base, qd + 2 * k, kd + 2 * k, idesc, k > 0 ? 1u : 0u);
        umma_commit(bar_s);
        ok = mbar_wait(bar_p, ph) && mbar_wait(bar_v, ph);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint64_t pd = make_desc(smem_u32(sP + s * kTileBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t vd = make_desc_mn(v_addr + (uint32_t)(s * 64 + k * 16) * 128u);
            umma(tmem_base + 128, pd + 2 * k, vd, idesc2, (s > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(bar_o);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int grow = qi * kAttT + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const float sc = p.scale * 1.4426950408889634f;       // scores in log2 units
    const uint32_t seed = p.drop_threshold ? *p.seed : 0u;
    const uint32_t drop_row = ((uint32_t)bh * (uint32_t)p.T + (uint32_t)grow) * (uint32_t)p.T;
    float m = -INFINITY, l = 0.f;
    float acc[kAttD];
#pragma unroll
    for (int d = 0; d < kAttD; ++d) acc[d] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int j = 0; j < nblk; ++j) {
      const uint32_t ph = (uint32_t)j & 1u;
      const float* kb = kbias + j * kAttT;
      ok = mbar_wait_warp(bar_s, ph);
      if (!ok) { *abort_flag = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float bm = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < kAttT; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) bm = fmaxf(bm, __uint_as_float(r[jj]) * sc + kb[c0 + jj]);
      }
      const float m_new = fmaxf(m, bm);
      const float mm = (m_new == -INFINITY) ? 0.f : m_new;  // a row with no valid key so far produces zeros, not NaN
      const float alpha = exp2f(m - mm);                    // 0 while the old maximum is -inf
      l *= alpha;
      m = m_new;
#pragma unroll 1
      for (int c0 = 0; c0 < kAttT; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float pv[32];
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const float e = exp2f(__uint_as_float(r[jj]) * sc + kb[c0 + jj] - mm);
          l += e;
          float keep = 1.f;
          if (p.drop_threshold) keep = att_hash(seed, drop_row + (uint32_t)(j * kAttT + c0 + jj)) >= p.drop_threshold ? p.keep_scale : 0.f;
          pv[jj] = e * keep;
        }
        uint8_t* tile = sP + (c0 >> 6) * kTileBytes;
#pragma unroll
        for (int v = 0; v < 4; ++v) store8_swz<T>(tile, row, ((c0 & 63) >> 3) + v, pv + v * 8);
      }
      fence_async_smem();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);
      ok = mbar_wait_warp(bar_o, ph);
      if (!ok) { *abort_flag = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < kAttD; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + (uint32_t)(128 + c0), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) acc[c0 + jj] = acc[c0 + jj] * alpha + __uint_as_float(r[jj]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (ok && grow < p.T) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* orow = static_cast<T*>(p.out) + ((int64_t)b * p.T + grow) * p.C + h * kAttD;
#pragma unroll
      for (int v = 0; v < kAttD / 8; ++v) {
        Vec16<T> o;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) o.v[jj] = Cvt<T>::from_f(acc[v * 8 + jj] * inv);
        st16(orow + v * 8, o);
      }
      const float mm = (m == -INFINITY) ? 0.f : m;
      if (p.lse) p.lse[((int64_t)b * p.heads + h) * p.T + grow] = (mm + log2f(fmaxf(l, 1e-30f))) * 0.6931471805599453f;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    // wait (bounded) for the bulk copies that may still be in flight before the shared memory is released
    mbar_wait(bar_q, 0);
    if (p.error_flag) atomicExch(p.error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ backward
// shared memory: K | V | Q0 | dO0 | Q1 | dO1 | P~ (2 key stages) | dS (2 key stages), key bias of the block, barriers.
// TMEM columns: S [0,128)  dP [128,256)  dV [256,320)  dQ of the block pair [320,384)  dK [384,448).
constexpr uint32_t kBwdLongSmem = 10 * kTileBytes + 128 * 4 + 1024 + 256;

template <typename T>
__global__ void __launch_bounds__(kAttThreads, 1)
attn_bwd_long_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const AttnParams p,
                     float* dq_part, int bf16) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;                 // stage s: Q at sQ + s * 2 tiles, dO one tile behind it
  uint8_t* sPt = smem + 6 * kTileBytes;
  uint8_t* sDS = smem + 8 * kTileBytes;
  float* kbias = reinterpret_cast<float*>(smem + 10 * kTileBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(kbias + 128);
  uint64_t* bar_kv = bars, *full = bars + 1, *empty = bars + 3, *bar_sdp = bars + 5, *bar_pd = bars + 6, *bar_out = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.T + kAttT - 1) / kAttT;
  const int kj = blockIdx.x % nblk;                    // key block of this CTA
  const int bh = blockIdx.x / nblk;
  const int b = bh / p.heads, h = bh % p.heads;
  constexpr uint32_t kTmemCols = 512;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1); mbar_init(&full[0], 1); mbar_init(&full[1], 1); mbar_init(&empty[0], 1); mbar_init(&empty[1], 1);
    mbar_init(bar_sdp, 1); mbar_init(bar_pd, 4); mbar_init(bar_out, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x >= 64 && threadIdx.x < 192) {
    const int k = threadIdx.x - 64;
    const int key = kj * kAttT + k;
    bool valid = key < p.T;
    if (valid && p.mask) valid = static_cast<const float*>(p.mask)[(int64_t)b * p.T + key] != 0.f;
    kbias[k] = valid ? 0.f : -INFINITY;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_kv, 2 * kTileBytes);
      tma_load_3d(sK, &map_qkv, p.C + h * kAttD, kj * kAttT, b, bar_kv);
      tma_load_3d(sV, &map_qkv, 2 * p.C + h * kAttD, kj * kAttT, b, bar_kv);
      for (int i = 0; i < nblk; ++i) {
        const int s = i & 1;
        if (i >= 2 && !mbar_wait(&empty[s], (uint32_t)((i >> 1) - 1) & 1u)) { *abort_flag = 1; break; }
        mbar_expect_tx(&full[s], 2 * kTileBytes);
        tma_load_3d(sQ + (size_t)s * 2 * kTileBytes, &map_qkv, h * kAttD, i * kAttT, b, &full[s]);
        tma_load_3d(sQ + (size_t)s * 2 * kTileBytes + kTileBytes, &map_do, h * kAttD, i * kAttT, b, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(bar_kv, 0);
      const uint32_t id_nn = make_idesc(bf16, 128, 0, 0);
      const uint32_t id_tt = make_idesc(bf16, kAttD, 1, 1);     // A MN-major (transposed view), B MN-major, N = 64
      const uint32_t id_nt = make_idesc(bf16, kAttD, 0, 1);     // A K-major, B MN-major
      const uint64_t kd = make_desc(smem_u32(sK)), vd = make_desc(smem_u32(sV));
      const uint32_t pt = smem_u32(sPt), ds = smem_u32(sDS), ka = smem_u32(sK);
      for (int i = 0; i < nblk && ok; ++i) {
        const int s = i & 1;
        const uint32_t qa = smem_u32(sQ + (size_t)s * 2 * kTileBytes), doa = qa + kTileBytes;
        ok = mbar_wait(&full[s], (uint32_t)(i >> 1) & 1u);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t qd = make_desc(qa), dd = make_desc(doa);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem_base, qd + 2 * k, kd + 2 * k, id_nn, k > 0 ? 1u : 0u);        // S = Q Kt
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem_base + 128, dd + 2 * k, vd + 2 * k, id_nn, k > 0 ? 1u : 0u);  // dP = dO Vt
        umma_commit(bar_sdp);
        ok = mbar_wait(bar_pd, (uint32_t)i & 1u);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t carry = i > 0 ? 1u : 0u;
        // dV[key, d] += sum_q P~[q, key] dO[q, d]: contraction over the 128 query rows, 16 at a time
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma(tmem_base + 256, make_desc_mn(pt + k * 2048u, kTileBytes), make_desc_mn(doa + k * 2048u), id_tt, (k > 0) ? 1u : carry);
        // dQ[q, d] = sum_key dS[q, key] K[key, d] over the keys of this block only
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2) {
          const uint64_t dsd = make_desc(ds + s2 * kTileBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma(tmem_base + 320, dsd + 2 * k, make_desc_mn(ka + (uint32_t)(s2 * 64 + k * 16) * 128u), id_nt, (s2 > 0 || k > 0) ? 1u : 0u);
        }
        // dK[key, d] += sum_q dS[q, key] Q[q, d]
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma(tmem_base + 384, make_desc_mn(ds + k * 2048u, kTileBytes), make_desc_mn(qa + k * 2048u), id_tt, (k > 0) ? 1u : carry);
        umma_commit(bar_out);
        umma_commit(&empty[s]);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const float sc = p.scale * 1.4426950408889634f;
    const uint32_t seed = p.drop_threshold ? *p.seed : 0u;
    bool ok = true;
#pragma unroll 1
    for (int i = 0; i < nblk; ++i) {
      const int grow = i * kAttT + row;
      const bool live = grow < p.T;
      // D = rowsum(dO * O) and the row's log-sum-exp, fetched while the tensor cores work
      float Dr = 0.f, lse2 = 0.f;
      if (live) {
        const T* orow = static_cast<const T*>(p.o) + ((int64_t)b * p.T + grow) * p.C + h * kAttD;
        const T* drow = static_cast<const T*>(p.dout) + ((int64_t)b * p.T + grow) * p.C + h * kAttD;
#pragma unroll
        for (int v = 0; v < kAttD / 8; ++v) {
          const Vec16<T> a = ld16(orow + v * 8), g = ld16(drow + v * 8);
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) Dr += Cvt<T>::to_f(a.v[jj]) * Cvt<T>::to_f(g.v[jj]);
        }
        lse2 = p.lse[((int64_t)b * p.heads + h) * p.T + grow] * 1.4426950408889634f;
      }
      ok = mbar_wait_warp(bar_sdp, (uint32_t)i & 1u);
      if (!ok) { *abort_flag = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t drop_base = ((uint32_t)bh * (uint32_t)p.T + (uint32_t)grow) * (uint32_t)p.T + (uint32_t)(kj * kAttT);
#pragma unroll 1
      for (int c0 = 0; c0 < kAttT; c0 += 32) {
        uint32_t rs[32], rd[32];
        tmem_ld32(lane_addr + (uint32_t)c0, rs);
        tmem_ld32(lane_addr + (uint32_t)(128 + c0), rd);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float ptv[32], dsv[32];
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const float e = live ? exp2f(__uint_as_float(rs[jj]) * sc + kbias[c0 + jj] - lse2) : 0.f;
          float keep = 1.f;
          if (p.drop_threshold) keep = att_hash(seed, drop_base + (uint32_t)(c0 + jj)) >= p.drop_threshold ? p.keep_scale : 0.f;
          ptv[jj] = e * keep;
          dsv[jj] = e * (__uint_as_float(rd[jj]) * keep - Dr) * p.scale;
        }
        uint8_t* t1 = sPt + (c0 >> 6) * kTileBytes;
        uint8_t* t2 = sDS + (c0 >> 6) * kTileBytes;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          store8_swz<T>(t1, row, ((c0 & 63) >> 3) + v, ptv + v * 8);
          store8_swz<T>(t2, row, ((c0 & 63) >> 3) + v, dsv + v * 8);
        }
      }
      fence_async_smem();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pd);
      ok = mbar_wait_warp(bar_out, (uint32_t)i & 1u);
      if (!ok) { *abort_flag = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float* slot = dq_part + (((int64_t)kj * p.N + b) * p.T + grow) * p.C + h * kAttD;
#pragma unroll 1
      for (int c0 = 0; c0 < kAttD; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + 320u + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (live) {
#pragma unroll
          for (int v = 0; v < 8; ++v)
            *reinterpret_cast<float4*>(slot + c0 + v * 4) = make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                                                                        __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (ok) {
      // dK and dV of this key block are complete with the last bar_out: accumulator row = key
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key = kj * kAttT + row;
      T* base = static_cast<T*>(p.dqkv) + ((int64_t)b * p.T + key) * 3 * p.C + h * kAttD;
#pragma unroll 1
      for (int part = 1; part < 3; ++part) {
        const uint32_t col = part == 1 ? 384u : 256u;          // dK, dV
        T* dst = base + (int64_t)part * p.C;
#pragma unroll 1
        for (int c0 = 0; c0 < kAttD; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(lane_addr + col + (uint32_t)c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (key < p.T) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              Vec16<T> o;
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) o.v[jj] = Cvt<T>::from_f(__uint_as_float(r[v * 8 + jj]));
              st16(dst + c0 + v * 8, o);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    mbar_wait(bar_kv, 0);
    if (p.error_flag) atomicExch(p.error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// dQ = sum over the key blocks' slots (fixed order), written into the Q third of the packed gradient.
template <typename T>
__global__ void attn_dq_finish_kernel(const float* __restrict__ dq_part, T* __restrict__ dqkv, int nblk, int64_t rows, int C) {
  const int64_t vecs = rows * (C / 8);
  const int64_t slot = rows * (int64_t)C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / (C / 8);
    const int c = (int)(i % (C / 8)) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < nblk; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(dq_part + k * slot + r * C + c);
      const float4 b = *reinterpret_cast<const float4*>(dq_part + k * slot + r * C + c + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(acc[j]);
    st16(dqkv + r * 3 * (int64_t)C + c, o);
  }
}

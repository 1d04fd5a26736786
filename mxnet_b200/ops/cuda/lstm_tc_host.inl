// Host side of lstm_tc.cu: shape plan, tensor maps, cooperative launches, exported entry points.
namespace mxb {

struct TcPlan {
  int ok;
  int U, KC, esz, Bp, Hp, C, Hc, KK;
  int stages_f, stages_b, stages_c;
  size_t smem_f, smem_b, smem_c;       // forward, backward, backward with the contraction cut over a cluster (0: does not fit)
};

constexpr size_t kTcSmemMax = 232448;                       // 227 KB per CTA
constexpr size_t kTcFixed = 1024 + 1024 + 16384;            // alignment, bookkeeping, slack behind the operands (see kernels)

static int tc_row_align(int H, int esz) {
  const long pitch = (long)H * esz;
  return pitch % 16 == 0 ? 16 : pitch % 8 == 0 ? 8 : pitch % 4 == 0 ? 4 : esz;
}

static TcPlan tc_plan(int dtype, int B, int H) {
  TcPlan pl = {};
  if (B < 1 || B > 128 || H < 1) return pl;
  pl.esz = dtype == kF32 ? 4 : 2;
  pl.U = dtype == kF32 ? 8 : 16;
  pl.KC = 128 / pl.esz;
  pl.Bp = (B + 7) / 8 * 8;
  pl.Hp = (H + pl.KC - 1) / pl.KC * pl.KC;
  pl.C = ((H + pl.U - 1) / pl.U + kTcCluster - 1) / kTcCluster * kTcCluster;      // whole clusters (idle CTAs own no unit)
  pl.Hc = pl.C * pl.U;
  pl.KK = 4 * pl.Hc;                                        // a multiple of KC for both element sizes
  if (pl.C > sm_count()) return pl;
  const size_t stage = (size_t)pl.Bp * 128;
  const size_t wf = (size_t)(pl.Hp / pl.KC) * 4 * pl.U * 128;
  const size_t wb = (size_t)(pl.KK / pl.KC) * pl.U * 128 + 2048;
  if (wf + kTcFixed + 3 * stage > kTcSmemMax || wb + kTcFixed + 3 * stage > kTcSmemMax) return pl;
  size_t sf = (kTcSmemMax - kTcFixed - wf) / stage, sb = (kTcSmemMax - kTcFixed - wb) / stage;
  pl.stages_f = (int)(sf > (size_t)kTcMaxStages ? (size_t)kTcMaxStages : sf);
  pl.stages_b = (int)(sb > (size_t)kTcMaxStages ? (size_t)kTcMaxStages : sb);
  pl.smem_f = wf + kTcFixed + (size_t)pl.stages_f * stage;
  pl.smem_b = wb + kTcFixed + (size_t)pl.stages_b * stage;
  // cluster variant of the backward pass: a quarter of the contraction axis per CTA, 4U units per cluster
  const size_t wc = (size_t)(pl.KK / kTcCluster / pl.KC) * kTcCluster * pl.U * 128;
  const size_t xc = (size_t)kTcCluster * 128 * pl.U * 4 + 64;
  if (wc + xc + kTcFixed + 3 * stage <= kTcSmemMax) {
    size_t sc = (kTcSmemMax - kTcFixed - wc - xc) / stage;
    pl.stages_c = (int)(sc > (size_t)kTcMaxStages ? (size_t)kTcMaxStages : sc);
    pl.smem_c = wc + xc + kTcFixed + (size_t)pl.stages_c * stage;
  }
  pl.ok = 1;
  return pl;
}

// Row-major [rows, cols] matrix of 16- or 32-bit elements; box = box_rows x 128 bytes, 128-byte swizzle.
static int tc_make_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  const int esz = dtype == kF32 ? 4 : 2;
  const CUtensorMapDataType ty = dtype == kF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * esz};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, ty, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

template <typename K>
static int tc_launch(K kernel, unsigned long long* seen, int grid, size_t smem, cudaStream_t st, const CUtensorMap& m0,
                     const CUtensorMap& m1, const LstmTcParams& p) {
  if (first_on_device(seen)) {
    cudaError_t rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemMax - 64);   // later shapes need more
    if (rc != cudaSuccess) return (int)rc;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;        // all CTAs resident at once: they meet at grid barriers
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, m0, m1, p);
}

// Backward with clusters of four: cooperative (grid barriers) and clustered launch.  Returns -100 when the device cannot
// hold all clusters at once (the caller then uses the plain kernel).
template <typename K>
static int tc_launch_cluster(K kernel, unsigned long long* seen, int grid, size_t smem, cudaStream_t st, const CUtensorMap& m0,
                             const CUtensorMap& m1, const LstmTcParams& p) {
  if (first_on_device(seen)) {
    cudaError_t rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemMax - 64);
    if (rc != cudaSuccess) return (int)rc;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kTcCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return -100; }
  if (clusters * kTcCluster < grid) return -100;
  return (int)cudaLaunchKernelEx(&cfg, kernel, m0, m1, p);
}

template <typename T, typename X, int U>
static int tc_backward_cluster(const TcPlan& pl, const CUtensorMap& md, const CUtensorMap& mw, LstmTcParams p, cudaStream_t st) {
  static unsigned long long seen = 0;
  p.stages = pl.stages_c;
  return tc_launch_cluster(lstm_tc_bwdc_kernel<T, X, U>, &seen, pl.C, pl.smem_c, st, md, mw, p);
}

static int g_tc_bwd_variant = 0;      // 0: cluster kernel where it fits, 1: plain kernel only

template <typename T, typename X, int U>
static int tc_forward(const TcPlan& pl, const CUtensorMap& mh, const CUtensorMap& mw, const LstmTcParams& p, cudaStream_t st) {
  static unsigned long long seen = 0;
  return tc_launch(lstm_tc_fwd_kernel<T, X, U>, &seen, pl.C, pl.smem_f, st, mh, mw, p);
}
template <typename T, typename X, int U>
static int tc_backward(const TcPlan& pl, const CUtensorMap& md, const CUtensorMap& mw, const LstmTcParams& p, cudaStream_t st) {
  static unsigned long long seen = 0;
  return tc_launch(lstm_tc_bwd_kernel<T, X, U>, &seen, pl.C, pl.smem_b, st, md, mw, p);
}

}  // namespace mxb

using namespace mxb;

// 1 when the tensor-core recurrence can run (dtype, batch, hidden size) on the current device.
MXB_EXPORT int mxb_lstm_tc_supported(int dtype, int B, int H) { return tc_plan(dtype, B, H).ok; }

// out[0..7] = U (units per CTA), Bp, Hp, C (CTAs), Hc, KK, forward ring depth, backward ring depth.
MXB_EXPORT int mxb_lstm_tc_dims(int dtype, int B, int H, int* out) {
  const TcPlan pl = tc_plan(dtype, B, H);
  if (!pl.ok) return -2;
  out[0] = pl.U; out[1] = pl.Bp; out[2] = pl.Hp; out[3] = pl.C; out[4] = pl.Hc; out[5] = pl.KK;
  out[6] = pl.stages_f; out[7] = pl.stages_b;
  return 0;
}

// Forward recurrence.  `xproj` [T, B, KK]: input projection with its columns in the per-CTA order.  `wp`: packed recurrent weights [C * 4U, Hp] in the element type (row c*4U + g*U + u = row
// g*H + c*U + u of W_hh, zero rows for units >= H, zero columns >= H).  `hbuf`: zero-initialised [2, Bp, Hp] elements.
// `gates` [T, B, KK] and `cs` [T, B, Hc] (fp32) are written when non-null.  `bar`: two zero-initialised words; bar[1] != 0
// afterwards means a wait timed out and the outputs are incomplete.
MXB_EXPORT int mxb_lstm_tc_forward(int dtype, const void* xproj, const void* wp, const void* h0, const void* c0, void* y, void* hT,
                                   void* cT, void* gates, void* cs, void* hbuf, void* bar, int T, int B, int H, void* stream) {
  const TcPlan pl = tc_plan(dtype, B, H);
  if (!pl.ok || T < 1) return -2;
  CUtensorMap mh, mw;
  int rc = tc_make_map(&mh, hbuf, dtype, 2 * (int64_t)pl.Bp, pl.Hp, pl.Bp);
  if (rc) return rc;
  rc = tc_make_map(&mw, wp, dtype, (int64_t)pl.C * 4 * pl.U, pl.Hp, 4 * pl.U);
  if (rc) return rc;
  LstmTcParams p = {};
  p.xproj = xproj; p.h0 = h0; p.c0 = c0; p.y = y; p.hT = hT; p.cT = cT; p.gates = gates; p.cs = (float*)cs; p.hbuf = hbuf;
  p.bar = (unsigned int*)bar;
  p.T = T; p.B = B; p.H = H; p.Bp = pl.Bp; p.Hp = pl.Hp; p.Hc = pl.Hc; p.KK = pl.KK; p.stages = pl.stages_f;
  p.yalign = tc_row_align(H, pl.esz);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) return tc_forward<float, float, 8>(pl, mh, mw, p, st);
  if (dtype == kF16) return tc_forward<__half, __half, 16>(pl, mh, mw, p, st);
  return tc_forward<__nv_bfloat16, __nv_bfloat16, 16>(pl, mh, mw, p, st);
}

// Backward recurrence.  `wb`: packed recurrent weights [C * U, KK]: row c*U + n holds column c*U + n of W_hh with the
// gate rows in the order of `gates` (zero for padded units).  `dgates` [T, B, KK] receives the gate gradients in that
// same column order (zero for padded units).
MXB_EXPORT int mxb_lstm_tc_backward(int dtype, const void* dy, const void* dhT, const void* dcT, const void* gates, const void* cs,
                                    const void* c0, const void* wb, void* dgates, void* dh0, void* dc0, void* bar,
                                    int T, int B, int H, void* stream) {
  const TcPlan pl = tc_plan(dtype, B, H);
  if (!pl.ok || T < 1) return -2;
  CUtensorMap md, mw;
  int rc = tc_make_map(&md, dgates, dtype, (int64_t)T * B, pl.KK, pl.Bp);
  if (rc) return rc;
  LstmTcParams p = {};
  p.dy = dy; p.dhT = dhT; p.dcT = dcT; p.gates = const_cast<void*>(gates); p.cs = (float*)const_cast<void*>(cs); p.c0 = c0;
  p.dgates = dgates; p.dh0 = dh0; p.dc0 = dc0; p.bar = (unsigned int*)bar;
  p.T = T; p.B = B; p.H = H; p.Bp = pl.Bp; p.Hp = pl.Hp; p.Hc = pl.Hc; p.KK = pl.KK; p.stages = pl.stages_b;
  p.yalign = tc_row_align(H, pl.esz);
  cudaStream_t st = (cudaStream_t)stream;
  if (pl.smem_c && g_tc_bwd_variant == 0) {
    rc = tc_make_map(&mw, wb, dtype, (int64_t)pl.C * pl.U, pl.KK, kTcCluster * pl.U);
    if (rc) return rc;
    rc = dtype == kF32 ? tc_backward_cluster<float, float, 8>(pl, md, mw, p, st)
         : dtype == kF16 ? tc_backward_cluster<__half, __half, 16>(pl, md, mw, p, st)
                         : tc_backward_cluster<__nv_bfloat16, __nv_bfloat16, 16>(pl, md, mw, p, st);
    if (rc != -100) return rc;
  }
  rc = tc_make_map(&mw, wb, dtype, (int64_t)pl.C * pl.U, pl.KK, pl.U);
  if (rc) return rc;
  if (dtype == kF32) return tc_backward<float, float, 8>(pl, md, mw, p, st);
  if (dtype == kF16) return tc_backward<__half, __half, 16>(pl, md, mw, p, st);
  return tc_backward<__nv_bfloat16, __nv_bfloat16, 16>(pl, md, mw, p, st);
}

// 0 (default): the backward pass cuts its contraction over clusters of four CTAs where they fit; 1: plain kernel only.
MXB_EXPORT void mxb_lstm_tc_set_backward_variant(int v) { g_tc_bwd_variant = v; }

// ---- GRU (gru_tc.inl) -------------------------------------------------------------------------------------------------------
namespace mxb {

struct GruPlan {
  int ok;
  int U, KC, esz, Bp, Hp, C, Hc, KK, NGP;
  int stages_f, stages_c;
  size_t smem_f, smem_c;
};

static GruPlan gru_plan(int dtype, int B, int H) {
  GruPlan pl = {};
  if (B < 1 || B > 128 || H < 1) return pl;
  pl.esz = dtype == kF32 ? 4 : 2;
  pl.U = dtype == kF32 ? 8 : 16;
  pl.KC = 128 / pl.esz;
  pl.NGP = pl.KC;                                            // 3U gate columns padded to one chunk
  pl.Bp = (B + 7) / 8 * 8;
  pl.Hp = (H + pl.KC - 1) / pl.KC * pl.KC;
  pl.C = ((H + pl.U - 1) / pl.U + kTcCluster - 1) / kTcCluster * kTcCluster;
  pl.Hc = pl.C * pl.U;
  pl.KK = pl.C * pl.NGP;
  if (pl.C > sm_count()) return pl;
  const size_t stage = (size_t)pl.Bp * 128;
  const size_t wf = (size_t)(pl.Hp / pl.KC) * pl.NGP * 128;
  const size_t wc = (size_t)(pl.KK / kTcCluster / pl.KC) * kTcCluster * pl.U * 128;
  const size_t xc = (size_t)kTcCluster * 128 * pl.U * 4 + 64;
  if (wf + kTcFixed + 3 * stage > kTcSmemMax || wc + xc + kTcFixed + 3 * stage > kTcSmemMax) return pl;
  size_t sf = (kTcSmemMax - kTcFixed - wf) / stage, sc = (kTcSmemMax - kTcFixed - wc - xc) / stage;
  pl.stages_f = (int)(sf > (size_t)kTcMaxStages ? (size_t)kTcMaxStages : sf);
  pl.stages_c = (int)(sc > (size_t)kTcMaxStages ? (size_t)kTcMaxStages : sc);
  pl.smem_f = wf + kTcFixed + (size_t)pl.stages_f * stage;
  pl.smem_c = wc + xc + kTcFixed + (size_t)pl.stages_c * stage;
  pl.ok = 1;
  return pl;
}

template <typename K>
static int gru_launch(K kernel, unsigned long long* seen, int grid, size_t smem, int cluster, cudaStream_t st, const CUtensorMap& m0,
                      const CUtensorMap& m1, const GruTcParams& p) {
  if (first_on_device(seen)) {
    cudaError_t rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemMax - 64);
    if (rc != cudaSuccess) return (int)rc;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeCooperative;
  attr[na].val.cooperative = 1;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (cluster > 1) {
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return -100; }
    if (clusters * cluster < grid) return -100;
  }
  return (int)cudaLaunchKernelEx(&cfg, kernel, m0, m1, p);
}

template <typename T, typename X, int U>
static int gru_forward(const GruPlan& pl, const CUtensorMap& mh, const CUtensorMap& mw, const GruTcParams& p, cudaStream_t st) {
  static unsigned long long seen = 0;
  return gru_launch(gru_tc_fwd_kernel<T, X, U>, &seen, pl.C, pl.smem_f, 1, st, mh, mw, p);
}
template <typename T, typename X, int U>
static int gru_backward(const GruPlan& pl, const CUtensorMap& md, const CUtensorMap& mw, const GruTcParams& p, cudaStream_t st) {
  static unsigned long long seen = 0;
  return gru_launch(gru_tc_bwdc_kernel<T, X, U>, &seen, pl.C, pl.smem_c, kTcCluster, st, md, mw, p);
}

// Whether the device holds all clusters of the backward kernel at once (its grid barrier needs every CTA resident).
template <typename K>
static bool gru_clusters_fit(K kernel, const GruPlan& pl) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemMax - 64) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.C);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = pl.smem_c;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kTcCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return false; }
  return clusters * kTcCluster >= pl.C;
}

}  // namespace mxb

// 1 when the tensor-core GRU recurrence can run (dtype, batch, hidden size) on the current device: the plan fits shared
// memory and the device holds every cluster of the backward kernel at the same time.
MXB_EXPORT int mxb_gru_tc_supported(int dtype, int B, int H) {
  const GruPlan pl = gru_plan(dtype, B, H);
  if (!pl.ok) return 0;
  if (dtype == kF32) return gru_clusters_fit(gru_tc_bwdc_kernel<float, float, 8>, pl) ? 1 : 0;
  if (dtype == kF16) return gru_clusters_fit(gru_tc_bwdc_kernel<__half, __half, 16>, pl) ? 1 : 0;
  return gru_clusters_fit(gru_tc_bwdc_kernel<__nv_bfloat16, __nv_bfloat16, 16>, pl) ? 1 : 0;
}

// out[0..6] = U, Bp, Hp, C, Hc, KK, NGP (padded gate columns per CTA).
MXB_EXPORT int mxb_gru_tc_dims(int dtype, int B, int H, int* out) {
  const GruPlan pl = gru_plan(dtype, B, H);
  if (!pl.ok) return -2;
  out[0] = pl.U; out[1] = pl.Bp; out[2] = pl.Hp; out[3] = pl.C; out[4] = pl.Hc; out[5] = pl.KK; out[6] = pl.NGP;
  return 0;
}

// Forward.  `xproj` [T, B, KK]: input projection in the per-CTA column order c*NGP + g*U + u (b_ih, plus b_hh for r and z).
// `wp` [C * NGP, Hp]: packed W_hh rows in the same order.  `bhn` [Hc] fp32: hidden-side bias of the candidate gate.
// `gates` [T, B, KK] and `hnb` [T, B, Hc] (fp32) are written when non-null.  `hbuf`: zero-initialised [2, Bp, Hp].
MXB_EXPORT int mxb_gru_tc_forward(int dtype, const void* xproj, const void* wp, const void* bhn, const void* h0, void* y, void* hT,
                                  void* gates, void* hnb, void* hbuf, void* bar, int T, int B, int H, void* stream) {
  const GruPlan pl = gru_plan(dtype, B, H);
  if (!pl.ok || T < 1) return -2;
  CUtensorMap mh, mw;
  int rc = tc_make_map(&mh, hbuf, dtype, 2 * (int64_t)pl.Bp, pl.Hp, pl.Bp);
  if (rc) return rc;
  rc = tc_make_map(&mw, wp, dtype, (int64_t)pl.C * pl.NGP, pl.Hp, pl.NGP);
  if (rc) return rc;
  GruTcParams g = {};
  LstmTcParams& p = g.base;
  p.xproj = xproj; p.y = y; p.hT = hT; p.gates = gates; p.hbuf = hbuf; p.bar = (unsigned int*)bar;
  p.T = T; p.B = B; p.H = H; p.Bp = pl.Bp; p.Hp = pl.Hp; p.Hc = pl.Hc; p.KK = pl.KK; p.stages = pl.stages_f;
  p.yalign = tc_row_align(H, pl.esz);
  g.bhn = bhn; g.hnb = (float*)hnb; g.h0 = h0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) return gru_forward<float, float, 8>(pl, mh, mw, g, st);
  if (dtype == kF16) return gru_forward<__half, __half, 16>(pl, mh, mw, g, st);
  return gru_forward<__nv_bfloat16, __nv_bfloat16, 16>(pl, mh, mw, g, st);
}

// Backward.  `wb` [Hc, KK]: row n = column n of W_hh with the gate rows in the order of `gates`.  `dgh` [T, B, KK] receives the
// hidden-side gate gradients (dar, daz, dan * r), `dgx` [T, B, KK] the input-side ones (dar, daz, dan).  Returns -100 when the
// device cannot hold all clusters at once.
MXB_EXPORT int mxb_gru_tc_backward(int dtype, const void* dy, const void* dhT, const void* gates, const void* hnb, const void* y,
                                   const void* h0, const void* wb, void* dgh, void* dgx, void* dh0, void* bar, int T, int B, int H,
                                   void* stream) {
  const GruPlan pl = gru_plan(dtype, B, H);
  if (!pl.ok || T < 1) return -2;
  CUtensorMap md, mw;
  int rc = tc_make_map(&md, dgh, dtype, (int64_t)T * B, pl.KK, pl.Bp);
  if (rc) return rc;
  rc = tc_make_map(&mw, wb, dtype, (int64_t)pl.C * pl.U, pl.KK, kTcCluster * pl.U);
  if (rc) return rc;
  GruTcParams g = {};
  LstmTcParams& p = g.base;
  p.dy = dy; p.dhT = dhT; p.gates = const_cast<void*>(gates); p.y = const_cast<void*>(y); p.dgates = dgh; p.dh0 = dh0;
  p.bar = (unsigned int*)bar;
  p.T = T; p.B = B; p.H = H; p.Bp = pl.Bp; p.Hp = pl.Hp; p.Hc = pl.Hc; p.KK = pl.KK; p.stages = pl.stages_c;
  p.yalign = tc_row_align(H, pl.esz);
  g.hnb = (float*)const_cast<void*>(hnb); g.dgx = dgx; g.h0 = h0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) return gru_backward<float, float, 8>(pl, md, mw, g, st);
  if (dtype == kF16) return gru_backward<__half, __half, 16>(pl, md, mw, g, st);
  return gru_backward<__nv_bfloat16, __nv_bfloat16, 16>(pl, md, mw, g, st);
}

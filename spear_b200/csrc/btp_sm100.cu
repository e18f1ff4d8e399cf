// libbtp_sm100.so - C ABI, argument checks, TMA descriptors and launches for the BTP kernels.
// Host-side counterpart of the reference's csrc/btp/_bindings.cu:19-229 and of the launchers
// csrc/btp/btp-forward.cu:462-527, csrc/btp/btp-backwards.cu:811-884; no torch types here.
#include "../../include/btp_sm100.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "btp_decode.cuh"
#include "btp_gated.cuh"
#include "btp_gated_bwd.cuh"
#include "btp_kernels.cuh"

namespace {

using namespace btp;

thread_local char tls_error[512] = "";
std::atomic<unsigned long long> g_launches{0};
std::atomic<unsigned long long> g_wait_limit_ns{btp::kWaitLimitNs};  // btp_sm100_set_wait_limit
std::atomic<unsigned int> g_test_missing_tx{0};                      // btp_sm100_test_expect_missing_bytes, one launch
std::atomic<int> g_seam_mode{BTP_SEAM_RECOMPUTE};                    // btp_sm100_set_seam_mode
thread_local int tls_last_grid = 0, tls_last_cluster = 0;            // btp_sm100_last_launch

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
  return code;
}

#define BTP_CUDA_TRY(expr)                                                                      \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess) return fail(BTP_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e));  \
  } while (0)

// ------------------------------------------------------------------ driver entry point for TMA descriptors
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

// Encoded descriptors, remembered per calling thread: a descriptor depends only on (base address, element type,
// rows, L, box), a training loop presents the same few tensors again and again, and encoding one costs about a
// microsecond of host time - as much as the rest of a call.  Thread-local, so no lock; 128 direct-mapped slots.
// (A descriptor holds no device state: reusing one for a buffer that was freed and allocated again at the same
// address with the same shape is correct.)
struct MapShape {
  int esz;       // element size: 2 (bf16) or 4 (float)
  int box_cols;  // box width in elements
  int box_rows;
  bool swizzle;  // 128-byte swizzle (the 16-row activation boxes) or none (single coefficient / dA rows)
};
constexpr MapShape kActBf16{2, 64, 16, true};   // x, y, dy, dx: [16 channels][64 tokens]
constexpr MapShape kActF32{4, 32, 16, true};    // float dy: [16 channels][32 tokens]
inline MapShape row_shape(int esz, int cols) { return MapShape{esz, cols, 1, false}; }  // one row of coeff / dA

struct MapCacheEntry {
  const void* base = nullptr;
  long long rows = 0;
  int L = 0;
  unsigned shape = 0;
  CUtensorMap map;
};
thread_local MapCacheEntry tls_maps[128];

int encode_map(CUtensorMap* map, const void* base, MapShape sh, long long rows, int L) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(BTP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(L), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(L) * sh.esz};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(sh.box_cols), static_cast<cuuint32_t>(sh.box_rows)};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = enc(map, sh.esz == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         sh.swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(BTP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return BTP_OK;
}

// Descriptor of a [rows][L] tensor read or written in boxes of shape `sh`.
int make_map(CUtensorMap* map, const void* base, MapShape sh, long long rows, int L) {
  const unsigned shape = static_cast<unsigned>(sh.esz) | static_cast<unsigned>(sh.box_cols) << 4 |
                         static_cast<unsigned>(sh.box_rows) << 16 | (sh.swizzle ? 1u << 24 : 0u);
  const uintptr_t h = (reinterpret_cast<uintptr_t>(base) >> 8) * 0x9E3779B97F4A7C15ull + shape * 0x85EBCA6Bu;
  MapCacheEntry& e = tls_maps[(h >> 40) & 127u];
  if (e.base == base && e.rows == rows && e.L == L && e.shape == shape) {
    *map = e.map;
    return BTP_OK;
  }
  const int rc = encode_map(map, base, sh, rows, L);
  if (rc) return rc;
  e.base = base; e.rows = rows; e.L = L; e.shape = shape; e.map = *map;
  return BTP_OK;
}

// Token-major tensor [B][L][cols] bf16 with row pitch `ld` elements; box = `box_rows` tokens x 64 channels.
// `narrow`: box = `box_rows` tokens x 16 channels (one head), dense 32-byte rows with the 32-byte swizzle - the per-head
// tiles of the kernels that read shared key/value heads in place.
int make_map_tokens(CUtensorMap* map, const void* base, int B, int L, int cols, long long ld, int box_rows = 64,
                    bool narrow = false) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(BTP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(L), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(ld) * 2 * L};
  const cuuint32_t box[3] = {narrow ? 16u : 64u, static_cast<cuuint32_t>(box_rows), 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, narrow ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(BTP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return BTP_OK;
}

// ------------------------------------------------------------------ per-device launch facts, computed once
struct DeviceInfo {
  bool ready = false;
  int sms = 0;
  int cc_major = 0;
};
DeviceInfo g_dev[64];
std::mutex g_dev_mutex;

int device_info(int* dev_out, DeviceInfo* info) {
  int dev = 0;
  BTP_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(BTP_ERR_CUDA, "device ordinal %d out of range", dev);
  // Binds the device's primary context to the calling thread: the descriptor encoder is a driver entry point
  // and threads that have made no runtime call yet (autograd's backward thread) have no current context.
  // Once per thread and device; later calls find the binding in place.
  thread_local int tls_bound_device = -1;
  thread_local DeviceInfo tls_info;
  if (tls_bound_device != dev) {
    BTP_CUDA_TRY(cudaSetDevice(dev));
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    if (!g_dev[dev].ready) {
      BTP_CUDA_TRY(cudaDeviceGetAttribute(&g_dev[dev].sms, cudaDevAttrMultiProcessorCount, dev));
      BTP_CUDA_TRY(cudaDeviceGetAttribute(&g_dev[dev].cc_major, cudaDevAttrComputeCapabilityMajor, dev));
      g_dev[dev].ready = true;
    }
    tls_info = g_dev[dev];
    tls_bound_device = dev;
  }
  *dev_out = dev;
  *info = tls_info;
  if (info->cc_major != 10) {
    return fail(BTP_ERR_UNSUPPORTED_DEVICE, "device %d has compute capability %d.x; this library is built for 10.x only",
                dev, info->cc_major);
  }
  return BTP_OK;
}

// One launchable kernel instance: sets its shared-memory limit and resident-CTA count once per device.
template <class KERNEL>
struct Launcher {
  KERNEL kernel;
  int smem_bytes;
  int threads;
  int warps;
  int ctas_per_sm[64];
  std::mutex mu;
  Launcher(KERNEL k, int smem, int nthreads) : kernel(k), smem_bytes(smem), threads(nthreads), warps(nthreads / 32) {
    for (int& c : ctas_per_sm) c = -1;
  }
  int prepare(int dev, int* ctas) {
    std::lock_guard<std::mutex> lock(mu);
    if (ctas_per_sm[dev] < 0) {
      BTP_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
      int occ = 0;
      BTP_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem_bytes));
      if (occ < 1) return fail(BTP_ERR_CUDA, "kernel does not fit on an SM (%d bytes of shared memory)", smem_bytes);
      ctas_per_sm[dev] = occ;
    }
    *ctas = ctas_per_sm[dev];
    return BTP_OK;
  }
  // persistent grid: every resident warp gets a contiguous share of the chunks
  int grid_for(int sms, int ctas, int total_chunks) const {
    long long want = (static_cast<long long>(total_chunks) + warps - 1) / warps;
    long long cap = static_cast<long long>(sms) * ctas;
    return static_cast<int>(want < cap ? want : cap);
  }
};

// Launch with programmatic stream serialization: the launch of this kernel is processed while the previous
// kernel of the stream still runs; its CTAs start when that kernel's CTAs have all exited and wait in pdl_wait()
// until its memory is visible.  That hides the launch latency (-2 % on the forward+backward step at
// B=1024, H=32, L=128).  The kernels do NOT release their successor early (griddepcontrol.launch_dependents at
// kernel start was measured 9 % slower: the successor's CTAs then occupy SMs while the stragglers finish;
// at the end of each warp's work it was measured within 0.6 % of not doing it).
// BTP_SM100_PDL=0 launches the plain way.
bool use_pdl() {
  static const bool v = [] {
    const char* e = getenv("BTP_SM100_PDL");
    return e ? atoi(e) != 0 : true;
  }();
  return v;
}

template <class... Params, class... Args>
cudaError_t launch_kernel(void (*kernel)(Params...), int grid, int threads, int smem_bytes, cudaStream_t stream,
                          const Args&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}

struct Dims {
  int B, H, L;
  long long BH;
  int ncs;
  int total_chunks;
};

int check_common(const char* fn, int B, int H, int L, int k, Dims* d) {
  if (B <= 0 || H <= 0 || L <= 0) return fail(BTP_ERR_BAD_SHAPE, "%s: B, H, L must be positive (got %d, %d, %d)", fn, B, H, L);
  if (L % 16 != 0) return fail(BTP_ERR_BAD_SHAPE, "%s: L must be a multiple of 16 (got %d)", fn, L);
  if (k != 1 && k != 2) return fail(BTP_ERR_BAD_ORDER, "%s: k must be 1 or 2 (got %d)", fn, k);
  d->B = B; d->H = H; d->L = L;
  d->BH = static_cast<long long>(B) * H;
  if (d->BH * 16 > 0x7fffffffll) return fail(BTP_ERR_BAD_SHAPE, "%s: B*H*16 = %lld rows exceeds the 2^31-1 limit", fn, d->BH * 16);
  return BTP_OK;
}

int set_chunks(const char* fn, Dims* d, int TL) {
  d->ncs = (d->L + TL - 1) / TL;
  const long long total = d->BH * d->ncs;
  if (total > 0x7fffffffll) return fail(BTP_ERR_BAD_SHAPE, "%s: %lld chunks exceed the 2^31-1 limit", fn, total);
  d->total_chunks = static_cast<int>(total);
  return BTP_OK;
}

// Whole sequences are dealt round-robin to the warps when they are numerous enough (at least 4 per warp) for
// that to balance; otherwise every warp takes a contiguous range of chunks.
bool use_interleave(const Dims& d, long long nwarps) { return d.BH >= 4 * nwarps; }

// Forward work distribution (RunCursor).  Measured on B200 over L = 256 ... 65536: dealing SHORT runs of chunks
// round-robin keeps the window of memory the whole GPU works on small, which HBM rewards more than the halo
// per run costs: runs of 2 chunks (256 tokens) beat whole sequences by 7-11 % at L = 1024 ... 4096 and a
// contiguous range per warp by up to 18 %; runs of 4 are 4 % better still around L = 8192; runs of 1 lose (a halo
// per chunk).  With an odd number of chunks per sequence whole sequences are dealt when there are at least 4 per
// warp.  Too few runs to balance (fewer than 4 per warp): one contiguous range per warp (run_len 0).
int forward_run_len(const Dims& d, long long nwarps) {
  const auto enough = [&](int r) { return static_cast<long long>(d.BH) * (d.ncs / r) >= 4 * nwarps; };
  if (d.ncs % 4 == 0 && d.ncs > 4 && d.L >= 8192 && d.L <= 16384 && enough(4)) return 4;
  if (d.ncs % 2 == 0 && enough(2)) return 2;
  if (enough(d.ncs)) return d.ncs;
  return 0;
}

bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

// ------------------------------------------------------------------ forward with the carry handed over between CTAs
// (BTP_SEAM_HANDOFF; see SeamLink in btp_kernels.cuh).  Applies when the forward would deal runs of at least two
// chunks, 2 ... 32 of them per sequence (a power of two): the warps of one sequence then form one cluster of
// runs_per_sequence / WARPS CTAs (1, 2, 4 or 8).  Returns BTP_OK with *done = false when the shape does not qualify
// and the caller has to take the recomputing kernel.
template <int COEF, bool F16>
int launch_forward_handoff(const void* coeff, const void* x, void* y, Dims d, cudaStream_t stream, bool* done) {
  constexpr int NBOX = 2, STAGES = 3, WARPS = 4;
  using LAYOUT = SmemLayout<COEF, NBOX, STAGES, WARPS, false, false, false>;
  constexpr int kSmem = LAYOUT::kBytes + WARPS * kSeamBytesPerWarp + kSeamBytesPerCta;
  auto kern = btp_forward_kernel<COEF, false, false, false, true, NBOX, STAGES, WARPS, F16, true>;
  static Launcher<decltype(kern)> L(kern, kSmem, WARPS * 32);
  *done = false;
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  int ctas;
  if ((rc = L.prepare(dev, &ctas))) return rc;
  if ((rc = set_chunks("btp_sm100_forward", &d, LAYOUT::kTL))) return rc;
  // the run length the recomputing kernel would take on the full grid decides, so that both walk memory alike
  const int run_len = forward_run_len(d, static_cast<long long>(info.sms) * ctas * WARPS);
  if (run_len < 2 || run_len >= d.ncs) return BTP_OK;
  const int rps = d.ncs / run_len;
  if (rps > 32 || (rps & (rps - 1)) != 0) return BTP_OK;
  const int cluster = rps > WARPS ? rps / WARPS : 1;
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // The grid is one wave: as many clusters as the device holds at once (fewer than SMs x CTAs per SM / cluster size
  // when the SMs of a GPC do not divide into clusters), asked once per device and cluster size.
  static int resident[64][4];  // [device][log2 cluster size], 0 = not asked yet
  static std::mutex resident_mu;
  const int slot = cluster == 1 ? 0 : cluster == 2 ? 1 : cluster == 4 ? 2 : 3;
  int clusters = 0;
  {
    std::lock_guard<std::mutex> lock(resident_mu);
    if (resident[dev][slot] == 0) {
      cfg.gridDim = dim3(static_cast<unsigned>(info.sms * ctas / cluster * cluster));
      cfg.numAttrs = 1;
      int n = 0;
      BTP_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
      if (n < 1) return fail(BTP_ERR_CUDA, "no cluster of %d CTAs fits on device %d", cluster, dev);
      resident[dev][slot] = n;
    }
    clusters = resident[dev][slot];
  }
  // a whole number of clusters; every warp of the grid has work (there are at least 4 runs per warp of the full grid)
  int grid = L.grid_for(info.sms, ctas, d.total_chunks / run_len);
  if (grid > clusters * cluster) grid = clusters * cluster;
  grid -= grid % cluster;
  if (grid < cluster) return BTP_OK;
  CUtensorMap tm_x, tm_y, tm_c;
  if ((rc = make_map(&tm_x, x, kActBf16, d.BH * 16, d.L))) return rc;
  if ((rc = make_map(&tm_y, y, kActBf16, d.BH * 16, d.L))) return rc;
  if ((rc = make_map(&tm_c, coeff, row_shape(CoefTraits<COEF>::kBytes, LAYOUT::kTL), d.BH, d.L))) return rc;
  KernelParams p{};
  p.coeff = coeff; p.x = x; p.out_f32 = y;
  p.L = d.L; p.ncs = d.ncs; p.total_chunks = d.total_chunks; p.use_carry = 1;
  p.run_len = run_len;
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  p.test_missing_tx = g_test_missing_tx.exchange(0u, std::memory_order_relaxed);
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.numAttrs = use_pdl() ? 2 : 1;
  BTP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tm_x, tm_y, tm_c, p));
  tls_last_grid = grid;
  tls_last_cluster = cluster;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  *done = true;
  return BTP_OK;
}

// ------------------------------------------------------------------ forward dispatch
template <int COEF, bool OUT_F32, bool CKPT, bool RAGGED, bool PRECISE, int NBOX, int STAGES, int WARPS, bool F16>
int launch_forward_impl(const void* coeff, const void* x, void* y, float* ckpt, Dims d, int k, cudaStream_t stream) {
  using LAYOUT = SmemLayout<COEF, NBOX, STAGES, WARPS, false, false, OUT_F32>;
  if constexpr (!OUT_F32 && !CKPT && !RAGGED && PRECISE && NBOX == 2 && STAGES == 3 && WARPS == 4) {
    if (k == 2 && g_seam_mode.load(std::memory_order_relaxed) == BTP_SEAM_HANDOFF) {
      bool done = false;
      const int rc = launch_forward_handoff<COEF, F16>(coeff, x, y, d, stream, &done);
      if (rc || done) return rc;
    }
  }
  auto kern = btp_forward_kernel<COEF, OUT_F32, CKPT, RAGGED, PRECISE, NBOX, STAGES, WARPS, F16>;
  static Launcher<decltype(kern)> L(kern, LAYOUT::kBytes, WARPS * 32);
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  int ctas;
  if ((rc = L.prepare(dev, &ctas))) return rc;
  if ((rc = set_chunks("btp_sm100_forward", &d, LAYOUT::kTL))) return rc;
  CUtensorMap tm_x, tm_y, tm_c;
  if ((rc = make_map(&tm_x, x, kActBf16, d.BH * 16, d.L))) return rc;
  if (OUT_F32) {
    tm_y = tm_x;  // unused by the kernel
  } else if ((rc = make_map(&tm_y, y, kActBf16, d.BH * 16, d.L))) {
    return rc;
  }
  if ((rc = make_map(&tm_c, coeff, row_shape(CoefTraits<COEF>::kBytes, LAYOUT::kTL), d.BH, d.L))) return rc;
  const int grid = L.grid_for(info.sms, ctas, d.total_chunks);
  KernelParams p{};
  p.coeff = coeff; p.x = x; p.out_f32 = y; p.ckpt = ckpt;
  p.L = d.L; p.ncs = d.ncs; p.total_chunks = d.total_chunks; p.use_carry = (k == 2);
  p.run_len = forward_run_len(d, static_cast<long long>(grid) * WARPS);
  p.interleave = p.run_len == d.ncs;
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  p.test_missing_tx = g_test_missing_tx.exchange(0u, std::memory_order_relaxed);
  BTP_CUDA_TRY(launch_kernel(kern, grid, WARPS * 32, LAYOUT::kBytes, stream, tm_x, tm_y, tm_c, p));
  tls_last_grid = grid;
  tls_last_cluster = 1;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BTP_OK;
}

// Sequences that are a whole number of chunks get the kernel without ragged-chunk handling.
template <int COEF, bool OUT_F32, bool CKPT, int NBOX, int STAGES, int WARPS, bool F16>
int launch_forward(const void* coeff, const void* x, void* y, float* ckpt, Dims d, int k, cudaStream_t stream) {
  const bool ragged = d.L % (64 * NBOX) != 0;
  if (!ragged) return launch_forward_impl<COEF, OUT_F32, CKPT, false, true, NBOX, STAGES, WARPS, F16>(coeff, x, y, ckpt, d, k, stream);
  return launch_forward_impl<COEF, OUT_F32, CKPT, true, true, NBOX, STAGES, WARPS, F16>(coeff, x, y, ckpt, d, k, stream);
}

// Launch shape of the forward kernel: 128-token chunks (2 boxes), 3 stages, 4 warps per CTA (16 warps per SM).
template <int COEF, bool OUT_F32, bool CKPT, bool F16>
int forward_variant(const void* coeff, const void* x, void* y, float* ckpt, Dims d, int k, cudaStream_t s) {
  return launch_forward<COEF, OUT_F32, CKPT, 2, 3, 4, F16>(coeff, x, y, ckpt, d, k, s);
}

template <int COEF, bool F16>
int forward_coef(const void* coeff, const void* x, void* y, float* ckpt, Dims d, int k, int out_dtype, cudaStream_t s) {
  const bool f32 = out_dtype == BTP_DTYPE_F32;
  const bool ck = ckpt != nullptr && k == 2;
  if (f32) return ck ? forward_variant<COEF, true, true, F16>(coeff, x, y, ckpt, d, k, s)
                     : forward_variant<COEF, true, false, F16>(coeff, x, y, ckpt, d, k, s);
  return ck ? forward_variant<COEF, false, true, F16>(coeff, x, y, ckpt, d, k, s)
            : forward_variant<COEF, false, false, F16>(coeff, x, y, ckpt, d, k, s);
}

// Decodes the dtype tags of a call: which 16-bit type the activations have, the coefficient's form, and whether
// the 16-bit output / upstream-gradient tag agrees with the activations.
struct Types {
  bool f16;    // activations (x, dx, a 16-bit y / dy / coefficient) are float16, else bfloat16
  int coef;    // kCoefBf16 (16-bit, in the activation type), kCoefF32, kCoefF32Log
};
int decode_types(const char* fn, int coeff_dtype, int io_dtype, const char* io_name, Types* t) {
  const int kind = coeff_dtype & 0xf;
  const bool flag = (coeff_dtype & BTP_ACT_F16) != 0;
  if ((coeff_dtype & ~(0xf | BTP_ACT_F16)) != 0 || kind > BTP_DTYPE_F16)
    return fail(BTP_ERR_BAD_DTYPE, "%s: unsupported coefficient dtype tag %d", fn, coeff_dtype);
  if (kind == BTP_DTYPE_BF16 && flag)
    return fail(BTP_ERR_BAD_DTYPE, "%s: a bfloat16 coefficient cannot go with float16 activations", fn);
  t->f16 = flag || kind == BTP_DTYPE_F16;
  t->coef = kind == BTP_DTYPE_F32 ? kCoefF32 : (kind == BTP_DTYPE_F32_LOG ? kCoefF32Log : kCoefBf16);
  const int same = t->f16 ? BTP_DTYPE_F16 : BTP_DTYPE_BF16;
  if (io_dtype != BTP_DTYPE_F32 && io_dtype != same)
    return fail(BTP_ERR_BAD_DTYPE, "%s: %s must be float32 or the activations' own 16-bit type (tag %d, got %d)", fn, io_name,
                same, io_dtype);
  return BTP_OK;
}

template <bool F16>
int forward_types(int coef, const void* coeff, const void* x, void* y, float* ckpt, Dims d, int k, int out_dtype, cudaStream_t s) {
  switch (coef) {
    case kCoefBf16: return forward_coef<kCoefBf16, F16>(coeff, x, y, ckpt, d, k, out_dtype, s);
    case kCoefF32: return forward_coef<kCoefF32, F16>(coeff, x, y, ckpt, d, k, out_dtype, s);
    default: return forward_coef<kCoefF32Log, F16>(coeff, x, y, ckpt, d, k, out_dtype, s);
  }
}

// ------------------------------------------------------------------ backward dispatch
template <int COEF, bool DY_F32, bool RAGGED, bool PRECISE, int NBOX, int STAGES, int WARPS, bool F16>
int launch_backward_impl(const void* coeff, const void* x, const void* dy, void* dx, float* dA, Dims d, int k,
                         cudaStream_t stream) {
  using LAYOUT = SmemLayout<COEF, NBOX, STAGES, WARPS, true, DY_F32>;
  auto kern = btp_backward_kernel<COEF, DY_F32, RAGGED, PRECISE, NBOX, STAGES, WARPS, F16>;
  static Launcher<decltype(kern)> L(kern, LAYOUT::kBytes, WARPS * 32);
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  int ctas;
  if ((rc = L.prepare(dev, &ctas))) return rc;
  if ((rc = set_chunks("btp_sm100_backward", &d, LAYOUT::kTL))) return rc;
  CUtensorMap tm_x, tm_dy, tm_dx, tm_c, tm_da;
  if ((rc = make_map(&tm_x, x, kActBf16, d.BH * 16, d.L))) return rc;
  if ((rc = make_map(&tm_dy, dy, DY_F32 ? kActF32 : kActBf16, d.BH * 16, d.L))) return rc;
  if ((rc = make_map(&tm_dx, dx, kActBf16, d.BH * 16, d.L))) return rc;
  if ((rc = make_map(&tm_c, coeff, row_shape(CoefTraits<COEF>::kBytes, LAYOUT::kTL), d.BH, d.L))) return rc;
  if ((rc = make_map(&tm_da, dA, row_shape(4, LAYOUT::kTL), d.BH, d.L))) return rc;
  const int grid = L.grid_for(info.sms, ctas, d.total_chunks);
  KernelParams p{};
  p.coeff = coeff; p.x = x; p.dy = dy; p.dA = dA;
  p.L = d.L; p.ncs = d.ncs; p.total_chunks = d.total_chunks; p.use_carry = (k == 2);
  p.interleave = use_interleave(d, static_cast<long long>(grid) * WARPS);
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  p.test_missing_tx = g_test_missing_tx.exchange(0u, std::memory_order_relaxed);
  BTP_CUDA_TRY(launch_kernel(kern, grid, WARPS * 32, LAYOUT::kBytes, stream, tm_x, tm_dy, tm_dx, tm_c, tm_da, p));
  tls_last_grid = grid;
  tls_last_cluster = 1;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BTP_OK;
}

template <int COEF, bool DY_F32, int NBOX, int STAGES, int WARPS, bool F16>
int launch_backward(const void* coeff, const void* x, const void* dy, void* dx, float* dA, Dims d, int k,
                    cudaStream_t stream) {
  const bool ragged = d.L % (64 * NBOX) != 0;
  if (!ragged) return launch_backward_impl<COEF, DY_F32, false, true, NBOX, STAGES, WARPS, F16>(coeff, x, dy, dx, dA, d, k, stream);
  return launch_backward_impl<COEF, DY_F32, true, true, NBOX, STAGES, WARPS, F16>(coeff, x, dy, dx, dA, d, k, stream);
}

// Launch shape of the backward kernel: 64-token chunks, 3 x-stages + 2 dy-stages, 4 warps per CTA.
template <int COEF, bool DY_F32, bool F16>
int backward_variant(const void* coeff, const void* x, const void* dy, void* dx, float* dA, Dims d, int k, cudaStream_t s) {
  return launch_backward<COEF, DY_F32, 1, 3, 4, F16>(coeff, x, dy, dx, dA, d, k, s);
}

template <bool F16>
int backward_types(int coef, bool f32, const void* coeff, const void* x, const void* dy, void* dx, float* dA, Dims d, int k,
                   cudaStream_t s) {
  switch (coef) {
    case kCoefBf16:
      return f32 ? backward_variant<kCoefBf16, true, F16>(coeff, x, dy, dx, dA, d, k, s)
                 : backward_variant<kCoefBf16, false, F16>(coeff, x, dy, dx, dA, d, k, s);
    case kCoefF32:
      return f32 ? backward_variant<kCoefF32, true, F16>(coeff, x, dy, dx, dA, d, k, s)
                 : backward_variant<kCoefF32, false, F16>(coeff, x, dy, dx, dA, d, k, s);
    default:
      return f32 ? backward_variant<kCoefF32Log, true, F16>(coeff, x, dy, dx, dA, d, k, s)
                 : backward_variant<kCoefF32Log, false, F16>(coeff, x, dy, dx, dA, d, k, s);
  }
}

// ------------------------------------------------------------------ gated forward launch
template <int TL, int STAGES, bool SHARED>
int launch_gated_forward(const void* a_logits, const void* b_logits, const void* c, const void* v, void* out, int B, int L,
                         int H, int kv_heads, long long ld_a, long long ld_b, long long ld_c, long long ld_v,
                         long long ld_out, int k, void* stream) {
  const char* fn = "btp_sm100_gated_forward";
  const long long cols = static_cast<long long>(H) * 16;
  const int hgs = H / 4;
  const int ncs = (L + TL - 1) / TL;
  const long long total = static_cast<long long>(B) * hgs * ncs;
  if (total > 0x7fffffffll) return fail(BTP_ERR_BAD_SHAPE, "%s: %lld work units exceed the 2^31-1 limit", fn, total);
  using SM = GatedSmem<TL, STAGES>;
  auto kern = btp_gated_forward_kernel<TL, STAGES, SHARED>;
  static Launcher<decltype(kern)> LN(kern, SM::kBytes, 128);
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  int ctas;
  if ((rc = LN.prepare(dev, &ctas))) return rc;
  CUtensorMap tm_b, tm_c, tm_v, tm_o;
  const int kv_cols = kv_heads * 16;
  if ((rc = make_map_tokens(&tm_b, b_logits, B, L, SHARED ? kv_cols : static_cast<int>(cols), ld_b, TL, SHARED))) return rc;
  if ((rc = make_map_tokens(&tm_c, c, B, L, SHARED ? kv_cols : static_cast<int>(cols), ld_c, TL, SHARED))) return rc;
  if ((rc = make_map_tokens(&tm_v, v, B, L, static_cast<int>(cols), ld_v, TL))) return rc;
  if ((rc = make_map_tokens(&tm_o, out, B, L, static_cast<int>(cols), ld_out, TL))) return rc;
  const long long cap = static_cast<long long>(info.sms) * ctas;
  const int grid = static_cast<int>(total < cap ? total : cap);
  GatedParams p{};
  p.a_logits = static_cast<const __nv_bfloat16*>(a_logits);
  p.b_logits = static_cast<const __nv_bfloat16*>(b_logits);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.ld_a = ld_a; p.ld_b = ld_b; p.ld_v = ld_v;
  p.L = L; p.H = H; p.hgs = hgs; p.ncs = ncs; p.total_units = static_cast<int>(total);
  p.use_carry = (k == 2);
  p.group = H / kv_heads;
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  p.interleave = static_cast<long long>(B) * hgs >= 3ll * grid;  // enough sequences to deal them out whole
  kern<<<grid, 128, SM::kBytes, static_cast<cudaStream_t>(stream)>>>(tm_b, tm_c, tm_v, tm_o, p);
  BTP_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BTP_OK;
}

// ------------------------------------------------------------------ gated backward launch
// Over how many neighbouring heads a CTA of the gated backward sums dB_logits / dC before storing them: the 4 heads
// of a CTA share one key/value head when the group size is a multiple of 4, form two pairs when it is 2.
int gated_backward_reduce(int H, int kv_heads) {
  const int group = H / kv_heads;
  return group % 4 == 0 ? 4 : (group == 2 ? 2 : 1);
}

template <bool SHARED, int REDUCE>
int launch_gated_backward(const void* a_logits, const void* b_logits, const void* c, const void* v, const void* dout,
                          void* da_logits, void* db_logits, void* dc, void* dv, int B, int L, int H, int kv_heads,
                          long long ld_a, long long ld_b, long long ld_c, long long ld_v, long long ld_do, long long ld_da,
                          long long ld_db, long long ld_dc, long long ld_dv, int k, void* stream) {
  const char* fn = "btp_sm100_gated_backward";
  const long long cols = static_cast<long long>(H) * 16;
  const int hgs = H / 4;
  const int ncs = (L + kGbTL - 1) / kGbTL;
  const long long total = static_cast<long long>(B) * hgs * ncs;
  if (total > 0x7fffffffll) return fail(BTP_ERR_BAD_SHAPE, "%s: %lld work units exceed the 2^31-1 limit", fn, total);
  constexpr int STAGES = 3;
  using SM = GatedBwdSmem<STAGES>;
  auto kern = btp_gated_backward_kernel<STAGES, SHARED, REDUCE>;
  static Launcher<decltype(kern)> LN(kern, SM::kBytes, 128);
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  int ctas;
  if ((rc = LN.prepare(dev, &ctas))) return rc;
  CUtensorMap tm_b, tm_c, tm_v, tm_do, tm_db, tm_dc, tm_dv;
  const int icols = static_cast<int>(cols), kcols = kv_heads * 16;
  // shared key/value heads: B_logits and C are read, and dB_logits / dC written, as per-head 16-column tiles
  if ((rc = make_map_tokens(&tm_b, b_logits, B, L, SHARED ? kcols : icols, ld_b, kGbTL, SHARED))) return rc;
  if ((rc = make_map_tokens(&tm_c, c, B, L, SHARED ? kcols : icols, ld_c, kGbTL, SHARED))) return rc;
  if ((rc = make_map_tokens(&tm_v, v, B, L, icols, ld_v, kGbTL))) return rc;
  if ((rc = make_map_tokens(&tm_do, dout, B, L, icols, ld_do, kGbTL))) return rc;
  constexpr int reduce = REDUCE;
  if ((rc = make_map_tokens(&tm_db, db_logits, B, L, icols / reduce, ld_db, kGbTL, SHARED))) return rc;
  if ((rc = make_map_tokens(&tm_dc, dc, B, L, icols / reduce, ld_dc, kGbTL, SHARED))) return rc;
  if ((rc = make_map_tokens(&tm_dv, dv, B, L, icols, ld_dv, kGbTL))) return rc;
  const long long cap = static_cast<long long>(info.sms) * ctas;
  const int grid = static_cast<int>(total < cap ? total : cap);
  GatedBwdParams p{};
  p.a_logits = static_cast<const __nv_bfloat16*>(a_logits);
  p.b_logits = static_cast<const __nv_bfloat16*>(b_logits);
  p.c = static_cast<const __nv_bfloat16*>(c);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.dout = static_cast<const __nv_bfloat16*>(dout);
  p.da_logits = static_cast<__nv_bfloat16*>(da_logits);
  p.ld_a = ld_a; p.ld_b = ld_b; p.ld_c = ld_c; p.ld_v = ld_v; p.ld_do = ld_do; p.ld_da = ld_da;
  p.L = L; p.H = H; p.hgs = hgs; p.ncs = ncs; p.total_units = static_cast<int>(total);
  p.use_carry = (k == 2);
  p.group = H / kv_heads;
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  p.interleave = static_cast<long long>(B) * hgs >= 3ll * grid;  // enough sequences to deal them out whole
  kern<<<grid, 128, SM::kBytes, static_cast<cudaStream_t>(stream)>>>(tm_b, tm_c, tm_v, tm_do, tm_db, tm_dc, tm_dv, p);
  BTP_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BTP_OK;
}

// ------------------------------------------------------------------ built-in scratch for btp_sm100_forward_noalloc
// Lives in the library image: every GPU that loads the library holds these 4 MiB until the process exits.
// `g_noalloc_ckpt` is only a host-side handle in host code; kernels get the device address that
// cudaGetSymbolAddress returns for the device that is current.
static __device__ __align__(256) float g_noalloc_ckpt[BTP_SM100_NOALLOC_MAX_HEAD_TOKENS];
float* g_noalloc_ckpt_addr[64];
std::mutex g_noalloc_mutex;

int noalloc_scratch(float** out) {
  int dev = 0;
  BTP_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(BTP_ERR_CUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ckpt_addr[dev] == nullptr) {
    float* ptr = nullptr;
    BTP_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_ckpt));
    if (ptr == nullptr) return fail(BTP_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the scratch array");
    g_noalloc_ckpt_addr[dev] = ptr;
  }
  *out = g_noalloc_ckpt_addr[dev];
  return BTP_OK;
}

}  // namespace

// ====================================================================== C ABI
namespace {
template <class T, class TA>
int launch_decode_step(const btp::DecodeParams& p, cudaStream_t s) {
  const long long quads = p.n_heads * 4;
  const long long blocks = (quads + 255) / 256;
  btp::btp_decode_step_kernel<T, TA><<<static_cast<unsigned>(blocks), 256, 0, s>>>(p);
  BTP_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BTP_OK;
}
template <class T, class TA>
int launch_prefill_state(const btp::PrefillStateParams& p, cudaStream_t s) {
  const long long threads = p.n_heads * 16;
  const long long blocks = (threads + 255) / 256;
  btp::btp_prefill_state_kernel<T, TA><<<static_cast<unsigned>(blocks), 256, 0, s>>>(p);
  BTP_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return BTP_OK;
}
bool bad_tag(int t) { return t != BTP_DTYPE_BF16 && t != BTP_DTYPE_F32; }
}  // namespace

extern "C" {

int btp_sm100_forward(const void* coeff, const void* x, void* y, float* checkpoint, int B, int H, int L, int k,
                      int coeff_dtype, int out_dtype, void* stream) {
  Dims d{};
  int rc = check_common("btp_sm100_forward", B, H, L, k, &d);
  if (rc) return rc;
  Types t{};
  if ((rc = decode_types("btp_sm100_forward", coeff_dtype, out_dtype, "y", &t))) return rc;
  if (!coeff || !x || !y) return fail(BTP_ERR_NULL_POINTER, "btp_sm100_forward: coeff, x and y must not be NULL");
  if (misaligned(coeff) || misaligned(x) || misaligned(y) || misaligned(checkpoint))
    return fail(BTP_ERR_MISALIGNED, "btp_sm100_forward: every pointer must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return t.f16 ? forward_types<true>(t.coef, coeff, x, y, checkpoint, d, k, out_dtype, s)
               : forward_types<false>(t.coef, coeff, x, y, checkpoint, d, k, out_dtype, s);
}

int btp_sm100_backward(const void* coeff, const void* x, const void* dy, const float* checkpoint, void* dx, float* dA,
                       int B, int H, int L, int k, int coeff_dtype, int dy_dtype, void* stream) {
  (void)checkpoint;  // the carry is recomputed; see the header
  Dims d{};
  int rc = check_common("btp_sm100_backward", B, H, L, k, &d);
  if (rc) return rc;
  Types t{};
  if ((rc = decode_types("btp_sm100_backward", coeff_dtype, dy_dtype, "dy", &t))) return rc;
  if (!coeff || !x || !dy || !dx || !dA)
    return fail(BTP_ERR_NULL_POINTER, "btp_sm100_backward: coeff, x, dy, dx and dA must not be NULL");
  if (misaligned(coeff) || misaligned(x) || misaligned(dy) || misaligned(dx) || misaligned(dA))
    return fail(BTP_ERR_MISALIGNED, "btp_sm100_backward: every pointer must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool f32 = dy_dtype == BTP_DTYPE_F32;
  return t.f16 ? backward_types<true>(t.coef, f32, coeff, x, dy, dx, dA, d, k, s)
               : backward_types<false>(t.coef, f32, coeff, x, dy, dx, dA, d, k, s);
}

int btp_sm100_forward_noalloc(const void* coeff, const void* x, void* y, int B, int H, int L, int k, int coeff_dtype,
                              int out_dtype, void* stream) {
  Dims d{};
  int rc = check_common("btp_sm100_forward_noalloc", B, H, L, k, &d);
  if (rc) return rc;
  Types t{};
  if ((rc = decode_types("btp_sm100_forward_noalloc", coeff_dtype, out_dtype, "y", &t))) return rc;
  if (!coeff || !x || !y) return fail(BTP_ERR_NULL_POINTER, "btp_sm100_forward_noalloc: coeff, x and y must not be NULL");
  if (misaligned(coeff) || misaligned(x) || misaligned(y))
    return fail(BTP_ERR_MISALIGNED, "btp_sm100_forward_noalloc: every pointer must be 16-byte aligned");
  // k == 1 has no carry and writes no record: the built-in array is not touched and its size does not matter
  if (k == 2 && d.BH * L > static_cast<long long>(BTP_SM100_NOALLOC_MAX_HEAD_TOKENS))
    return fail(BTP_ERR_TOO_LARGE,
                "btp_sm100_forward_noalloc: B*H*L = %lld exceeds the built-in scratch of %d head-tokens; "
                "call btp_sm100_forward with a checkpoint buffer of your own",
                d.BH * L, BTP_SM100_NOALLOC_MAX_HEAD_TOKENS);
  {
    int dev;
    DeviceInfo info;
    if ((rc = device_info(&dev, &info))) return rc;  // an unsupported device is reported as such, not as a failed lookup
  }
  float* scratch = nullptr;
  if (k == 2 && (rc = noalloc_scratch(&scratch))) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return t.f16 ? forward_types<true>(t.coef, coeff, x, y, scratch, d, k, out_dtype, s)
               : forward_types<false>(t.coef, coeff, x, y, scratch, d, k, out_dtype, s);
}

int btp_sm100_gated_forward(const void* a_logits, const void* b_logits, const void* c, const void* v, void* out, int B,
                            int L, int H, int kv_heads, long long ld_a, long long ld_b, long long ld_c, long long ld_v,
                            long long ld_out, int k, void* stream) {
  const char* fn = "btp_sm100_gated_forward";
  if (B <= 0 || H <= 0 || L <= 0) return fail(BTP_ERR_BAD_SHAPE, "%s: B, L, H must be positive (got %d, %d, %d)", fn, B, L, H);
  if (L % 16 != 0) return fail(BTP_ERR_BAD_SHAPE, "%s: L must be a multiple of 16 (got %d)", fn, L);
  if (H % 4 != 0) return fail(BTP_ERR_BAD_SHAPE, "%s: the number of heads must be a multiple of 4 (got %d)", fn, H);
  if (k != 1 && k != 2) return fail(BTP_ERR_BAD_ORDER, "%s: k must be 1 or 2 (got %d)", fn, k);
  if (!a_logits || !b_logits || !c || !v || !out) return fail(BTP_ERR_NULL_POINTER, "%s: no pointer may be NULL", fn);
  if (kv_heads <= 0 || H % kv_heads != 0)
    return fail(BTP_ERR_BAD_SHAPE, "%s: kv_heads must divide the number of heads (got %d, %d)", fn, kv_heads, H);
  const long long cols = static_cast<long long>(H) * 16, kcols = static_cast<long long>(kv_heads) * 16;
  if (ld_a < H || ld_b < kcols || ld_c < kcols || ld_v < cols || ld_out < cols)
    return fail(BTP_ERR_BAD_SHAPE, "%s: a row pitch is smaller than its row", fn);
  if (ld_b % 8 || ld_c % 8 || ld_v % 8 || ld_out % 8)
    return fail(BTP_ERR_MISALIGNED, "%s: row pitches of B_logits, C, V and out must be multiples of 8 elements", fn);
  if (misaligned(b_logits) || misaligned(c) || misaligned(v) || misaligned(out) || (reinterpret_cast<uintptr_t>(a_logits) & 1u))
    return fail(BTP_ERR_MISALIGNED, "%s: B_logits, C, V and out must be 16-byte aligned", fn);
  // Measured on B200: 32-token chunks (6 CTAs per SM) are 5-7 % faster than 64-token chunks (3 CTAs per SM) as
  // long as whole sequences can still be dealt round-robin to the larger grid and the sequences are short;
  // with few or long sequences the 64-token kernel wins (by up to 28 % at L = 2048 with 2048 head groups).
  int dev;
  DeviceInfo info;
  const int rc = device_info(&dev, &info);
  if (rc) return rc;
  const long long head_groups = static_cast<long long>(B) * (H / 4);
  const bool small = L <= 512 && head_groups >= 3ll * 6 * info.sms;
  if (kv_heads < H)
    return small ? launch_gated_forward<32, 3, true>(a_logits, b_logits, c, v, out, B, L, H, kv_heads, ld_a, ld_b, ld_c, ld_v, ld_out, k, stream)
                 : launch_gated_forward<64, 3, true>(a_logits, b_logits, c, v, out, B, L, H, kv_heads, ld_a, ld_b, ld_c, ld_v, ld_out, k, stream);
  return small ? launch_gated_forward<32, 3, false>(a_logits, b_logits, c, v, out, B, L, H, kv_heads, ld_a, ld_b, ld_c, ld_v, ld_out, k, stream)
               : launch_gated_forward<64, 3, false>(a_logits, b_logits, c, v, out, B, L, H, kv_heads, ld_a, ld_b, ld_c, ld_v, ld_out, k, stream);
}

int btp_sm100_gated_backward(const void* a_logits, const void* b_logits, const void* c, const void* v, const void* dout,
                             void* da_logits, void* db_logits, void* dc, void* dv, int B, int L, int H, int kv_heads,
                             long long ld_a, long long ld_b, long long ld_c, long long ld_v, long long ld_do,
                             long long ld_da, long long ld_db, long long ld_dc, long long ld_dv, int k, void* stream) {
  const char* fn = "btp_sm100_gated_backward";
  if (B <= 0 || H <= 0 || L <= 0) return fail(BTP_ERR_BAD_SHAPE, "%s: B, L, H must be positive (got %d, %d, %d)", fn, B, L, H);
  if (L % 16 != 0) return fail(BTP_ERR_BAD_SHAPE, "%s: L must be a multiple of 16 (got %d)", fn, L);
  if (H % 4 != 0) return fail(BTP_ERR_BAD_SHAPE, "%s: the number of heads must be a multiple of 4 (got %d)", fn, H);
  if (k != 1 && k != 2) return fail(BTP_ERR_BAD_ORDER, "%s: k must be 1 or 2 (got %d)", fn, k);
  if (!a_logits || !b_logits || !c || !v || !dout || !da_logits || !db_logits || !dc || !dv)
    return fail(BTP_ERR_NULL_POINTER, "%s: no pointer may be NULL", fn);
  if (kv_heads <= 0 || H % kv_heads != 0)
    return fail(BTP_ERR_BAD_SHAPE, "%s: kv_heads must divide the number of heads (got %d, %d)", fn, kv_heads, H);
  const long long cols = static_cast<long long>(H) * 16, kcols = static_cast<long long>(kv_heads) * 16;
  const long long gcols = cols / gated_backward_reduce(H, kv_heads);  // width of dB_logits and dC (see the header)
  if (ld_a < H || ld_da < H || ld_b < kcols || ld_c < kcols || ld_v < cols || ld_do < cols || ld_db < gcols || ld_dc < gcols ||
      ld_dv < cols)
    return fail(BTP_ERR_BAD_SHAPE, "%s: a row pitch is smaller than its row", fn);
  if (ld_b % 8 || ld_c % 8 || ld_v % 8 || ld_do % 8 || ld_db % 8 || ld_dc % 8 || ld_dv % 8 || ld_da % 4)
    return fail(BTP_ERR_MISALIGNED, "%s: row pitches must be multiples of 8 elements (dA_logits: 4)", fn);
  if (misaligned(b_logits) || misaligned(c) || misaligned(v) || misaligned(dout) || misaligned(db_logits) || misaligned(dc) ||
      misaligned(dv) || (reinterpret_cast<uintptr_t>(a_logits) & 1u) || (reinterpret_cast<uintptr_t>(da_logits) & 7u))
    return fail(BTP_ERR_MISALIGNED, "%s: the [B,L,H*16] tensors must be 16-byte aligned, dA_logits 8-byte aligned", fn);
#define BTP_GATED_BWD(SHARED, REDUCE)                                                                                  \
  launch_gated_backward<SHARED, REDUCE>(a_logits, b_logits, c, v, dout, da_logits, db_logits, dc, dv, B, L, H, kv_heads, \
                                        ld_a, ld_b, ld_c, ld_v, ld_do, ld_da, ld_db, ld_dc, ld_dv, k, stream)
  if (kv_heads == H) return BTP_GATED_BWD(false, 1);
  switch (gated_backward_reduce(H, kv_heads)) {
    case 4: return BTP_GATED_BWD(true, 4);
    case 2: return BTP_GATED_BWD(true, 2);
    default: return BTP_GATED_BWD(true, 1);
  }
#undef BTP_GATED_BWD
}

int btp_sm100_decode_step(const void* a_t, const void* x_t, const void* c_t, const void* v_t, void* y_t,
                          const void* h_loc, const void* r_pref, const void* c_prev_loc, void* h_loc_out,
                          void* r_pref_out, void* c_prev_loc_out, long long n_heads, int block_complete,
                          int gate_is_log, int r_is_log, int dtype, int gate_dtype, void* stream) {
  const char* fn = "btp_sm100_decode_step";
  if (n_heads <= 0 || n_heads > (1ll << 40)) return fail(BTP_ERR_BAD_SHAPE, "%s: n_heads must be in [1, 2^40] (got %lld)", fn, n_heads);
  if (bad_tag(dtype) || bad_tag(gate_dtype))
    return fail(BTP_ERR_BAD_DTYPE, "%s: dtype and gate_dtype must be BTP_DTYPE_BF16 or BTP_DTYPE_F32", fn);
  if (!a_t || !x_t || !c_t || !v_t || !y_t || !h_loc || !c_prev_loc || !h_loc_out || !r_pref_out)
    return fail(BTP_ERR_NULL_POINTER, "%s: only r_pref and (unless the block completes) c_prev_loc_out may be NULL", fn);
  if (block_complete && !c_prev_loc_out)
    return fail(BTP_ERR_NULL_POINTER, "%s: c_prev_loc_out is needed on the step that completes a block", fn);
  if (misaligned(x_t) || misaligned(c_t) || misaligned(v_t) || misaligned(y_t) || misaligned(h_loc) || misaligned(c_prev_loc) ||
      misaligned(h_loc_out) || (c_prev_loc_out && misaligned(c_prev_loc_out)))
    return fail(BTP_ERR_MISALIGNED, "%s: the [n_heads,16] tensors must be 16-byte aligned", fn);
  const unsigned amask = gate_dtype == BTP_DTYPE_F32 ? 3u : 1u;
  if ((reinterpret_cast<uintptr_t>(a_t) & amask) || (reinterpret_cast<uintptr_t>(r_pref_out) & amask) ||
      (r_pref && (reinterpret_cast<uintptr_t>(r_pref) & amask)))
    return fail(BTP_ERR_MISALIGNED, "%s: a gate pointer is not aligned to its element size", fn);
  if ((n_heads * 4 + 255) / 256 > 0x7fffffffll) return fail(BTP_ERR_BAD_SHAPE, "%s: too many heads for one launch", fn);
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  btp::DecodeParams p{};
  p.a = a_t; p.x = x_t; p.c = c_t; p.v = v_t; p.y = y_t;
  p.h_in = h_loc; p.r_in = r_pref; p.cprev = c_prev_loc;
  p.h_out = h_loc_out; p.r_out = r_pref_out; p.cprev_out = c_prev_loc_out;
  p.n_heads = n_heads;
  p.a_log = gate_is_log != 0;
  p.r_log = r_is_log != 0;
  p.block_done = block_complete != 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == BTP_DTYPE_BF16)
    return gate_dtype == BTP_DTYPE_BF16 ? launch_decode_step<__nv_bfloat16, __nv_bfloat16>(p, s)
                                        : launch_decode_step<__nv_bfloat16, float>(p, s);
  return gate_dtype == BTP_DTYPE_BF16 ? launch_decode_step<float, __nv_bfloat16>(p, s) : launch_decode_step<float, float>(p, s);
}

int btp_sm100_prefill_state(const void* a, const void* x, void* h_loc, void* r_pref, void* c_prev_loc, long long n_heads,
                            int L, int gate_is_log, int dtype, int gate_dtype, void* stream) {
  const char* fn = "btp_sm100_prefill_state";
  if (n_heads <= 0 || L <= 0 || n_heads > (1ll << 36))
    return fail(BTP_ERR_BAD_SHAPE, "%s: n_heads and L must be positive (got %lld, %d)", fn, n_heads, L);
  if (bad_tag(dtype) || bad_tag(gate_dtype))
    return fail(BTP_ERR_BAD_DTYPE, "%s: dtype and gate_dtype must be BTP_DTYPE_BF16 or BTP_DTYPE_F32", fn);
  if (!a || !x || !h_loc || !r_pref || !c_prev_loc) return fail(BTP_ERR_NULL_POINTER, "%s: no pointer may be NULL", fn);
  const unsigned xmask = dtype == BTP_DTYPE_F32 ? 3u : 1u;
  const unsigned amask = gate_dtype == BTP_DTYPE_F32 ? 3u : 1u;
  if ((reinterpret_cast<uintptr_t>(x) & xmask) || (reinterpret_cast<uintptr_t>(h_loc) & xmask) ||
      (reinterpret_cast<uintptr_t>(c_prev_loc) & xmask) || (reinterpret_cast<uintptr_t>(a) & amask) ||
      (reinterpret_cast<uintptr_t>(r_pref) & amask))
    return fail(BTP_ERR_MISALIGNED, "%s: a pointer is not aligned to its element size", fn);
  if ((n_heads * 16 + 255) / 256 > 0x7fffffffll) return fail(BTP_ERR_BAD_SHAPE, "%s: too many heads for one launch", fn);
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  btp::PrefillStateParams p{};
  p.a = a; p.x = x; p.h_loc = h_loc; p.r_pref = r_pref; p.cprev = c_prev_loc;
  p.n_heads = n_heads; p.L = L; p.a_log = gate_is_log != 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == BTP_DTYPE_BF16)
    return gate_dtype == BTP_DTYPE_BF16 ? launch_prefill_state<__nv_bfloat16, __nv_bfloat16>(p, s)
                                        : launch_prefill_state<__nv_bfloat16, float>(p, s);
  return gate_dtype == BTP_DTYPE_BF16 ? launch_prefill_state<float, __nv_bfloat16>(p, s) : launch_prefill_state<float, float>(p, s);
}

int btp_sm100_noalloc_read_record(float* dst, long long n_floats, void* stream) {
  const char* fn = "btp_sm100_noalloc_read_record";
  if (!dst) return fail(BTP_ERR_NULL_POINTER, "%s: dst must not be NULL", fn);
  if (n_floats <= 0 || n_floats > static_cast<long long>(BTP_SM100_NOALLOC_MAX_HEAD_TOKENS))
    return fail(BTP_ERR_BAD_SHAPE, "%s: n_floats must be in [1, %d] (got %lld)", fn, BTP_SM100_NOALLOC_MAX_HEAD_TOKENS, n_floats);
  int dev;
  DeviceInfo info;
  int rc = device_info(&dev, &info);
  if (rc) return rc;
  float* scratch = nullptr;
  if ((rc = noalloc_scratch(&scratch))) return rc;
  BTP_CUDA_TRY(cudaMemcpyAsync(dst, scratch, static_cast<size_t>(n_floats) * sizeof(float), cudaMemcpyDeviceToDevice,
                               static_cast<cudaStream_t>(stream)));
  return BTP_OK;
}

unsigned long long btp_sm100_set_wait_limit(unsigned long long ns) {
  return g_wait_limit_ns.exchange(ns ? ns : btp::kWaitLimitNs, std::memory_order_relaxed);
}

int btp_sm100_set_seam_mode(int mode) {
  if (mode != BTP_SEAM_RECOMPUTE && mode != BTP_SEAM_HANDOFF) return g_seam_mode.load(std::memory_order_relaxed);
  return g_seam_mode.exchange(mode, std::memory_order_relaxed);
}

void btp_sm100_last_launch(int* grid, int* cluster) {
  if (grid) *grid = tls_last_grid;
  if (cluster) *cluster = tls_last_cluster;
}

void btp_sm100_test_expect_missing_bytes(unsigned int bytes) { g_test_missing_tx.store(bytes, std::memory_order_relaxed); }

const char* btp_sm100_status_string(int status) {
  switch (status) {
    case BTP_OK: return "BTP_OK";
    case BTP_ERR_NULL_POINTER: return "BTP_ERR_NULL_POINTER";
    case BTP_ERR_BAD_SHAPE: return "BTP_ERR_BAD_SHAPE";
    case BTP_ERR_BAD_ORDER: return "BTP_ERR_BAD_ORDER";
    case BTP_ERR_BAD_DTYPE: return "BTP_ERR_BAD_DTYPE";
    case BTP_ERR_MISALIGNED: return "BTP_ERR_MISALIGNED";
    case BTP_ERR_CUDA: return "BTP_ERR_CUDA";
    case BTP_ERR_UNSUPPORTED_DEVICE: return "BTP_ERR_UNSUPPORTED_DEVICE";
    case BTP_ERR_DEVICE_TIMEOUT: return "BTP_ERR_DEVICE_TIMEOUT";
    case BTP_ERR_TOO_LARGE: return "BTP_ERR_TOO_LARGE";
    default: return "BTP_ERR_UNKNOWN";
  }
}

const char* btp_sm100_last_error(void) { return tls_error; }

int btp_sm100_device_status(void* stream, unsigned int* detail) {
  BTP_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  unsigned int words[4] = {0, 0, 0, 0};
  BTP_CUDA_TRY(cudaMemcpyFromSymbol(words, btp::g_btp_device_error, sizeof(words)));
  if (detail) memcpy(detail, words, sizeof(words));
  if (words[0] == 0) return BTP_OK;
  const unsigned int zero[4] = {0, 0, 0, 0};
  BTP_CUDA_TRY(cudaMemcpyToSymbol(btp::g_btp_device_error, zero, sizeof(zero)));
  return fail(BTP_ERR_DEVICE_TIMEOUT, "%s: block %u warp %u chunk %u",
              words[0] == 2 ? "shared-memory base not 1024-byte aligned" : "a kernel wait gave up", words[1], words[2],
              words[3]);
}

unsigned long long btp_sm100_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int btp_sm100_abi_version(void) { return BTP_SM100_ABI_VERSION; }

}  // extern "C"

// C ABI of the library: argument validation, TMA tensor maps, tile / split-K
// selection and kernel launches.  Validation comes first in every entry point
// and touches no CUDA state, so wrong calls are rejected the same way with or
// without a GPU in the machine.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>

#include <dlfcn.h>

#include "tg_internal.h"

namespace tg {
namespace {

thread_local char g_err[512] = "";

int32_t fail(int32_t rc, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return rc;
}

// Device status word written by a kernel whose bounded wait expired.
__device__ int32_t g_status_word;

constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  int num_sms = 0;
  int32_t* status = nullptr;
};
DeviceState g_dev[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != dev) {
      err = cudaSetDevice(dev);
      changed = (err == cudaSuccess);
    }
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};

// Called with `dev` current.
int32_t init_device(int dev) {
  if (dev < 0 || dev >= kMaxDevices) return fail(TG_ERR_DEVICE, "device id %d out of range", dev);
  DeviceState& st = g_dev[dev];
  if (st.ready) return TG_OK;
  int major = 0, minor = 0, sms = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot query CUDA device %d (is there a GPU?)", dev);
  }
  if (major != 10) return fail(TG_ERR_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev, major, minor);
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fn == nullptr) {
      cudaGetLastError();
      return fail(TG_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  void* sp = nullptr;
  if (cudaGetSymbolAddress(&sp, g_status_word) != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot resolve the status word on device %d", dev);
  }
  st.status = static_cast<int32_t*>(sp);
  st.num_sms = sms;
  st.ready = true;
  return TG_OK;
}

// Tuning / debug knobs come from TILEGYM_B200_* environment variables.  They are read ONCE, on the first call that
// needs one (a dozen getenv scans per GEMM launch cost more than a decode kernel's set-up), and again whenever
// tg_reload_env() is called (tests flip knobs between calls).
enum Knob : int {
  kKnobSplits, kKnobTileRows, kKnobForcePath, kKnobPairMinTiles, kKnob2Cta, kKnobBn, kKnobSmallmWs, kKnobPdl,
  kKnobStaticWeights, kKnobGroupM, kKnobTailDiv, kKnobTmaStore, kKnobBsWideMin, kKnobBsWide,
  kKnobBsSmallm, kKnobGroupOrder, kKnobQuantFused, kKnobGroupedSmallm, kKnobCount
};
const char* const kKnobNames[kKnobCount] = {
    "TILEGYM_B200_SPLITS", "TILEGYM_B200_TILE_ROWS", "TILEGYM_B200_FORCE_PATH", "TILEGYM_B200_PAIR_MIN_TILES",
    "TILEGYM_B200_2CTA", "TILEGYM_B200_BN", "TILEGYM_B200_SMALLM_WS", "TILEGYM_B200_PDL",
    "TILEGYM_B200_STATIC_WEIGHTS", "TILEGYM_B200_GROUP_M", "TILEGYM_B200_TAIL_DIV", "TILEGYM_B200_TMA_STORE",
    "TILEGYM_B200_BS_WIDE_MIN", "TILEGYM_B200_BS_WIDE", "TILEGYM_B200_BS_SMALLM", "TILEGYM_B200_GROUP_ORDER", "TILEGYM_B200_QUANT_FUSED",
    "TILEGYM_B200_GROUPED_SMALLM"};
struct KnobTable {
  bool loaded = false;
  bool present[kKnobCount] = {};
  int value[kKnobCount] = {};
  int force_path = 0;  // TILEGYM_B200_FORCE_PATH: 0 unset, 1 "gemm", 2 "smallm"
};
KnobTable g_knobs;

void load_knobs() {
  for (int i = 0; i < kKnobCount; ++i) {
    const char* v = getenv(kKnobNames[i]);
    g_knobs.present[i] = v != nullptr && *v != 0;
    g_knobs.value[i] = g_knobs.present[i] ? atoi(v) : 0;
  }
  const char* f = getenv(kKnobNames[kKnobForcePath]);
  g_knobs.force_path = (f && !strcmp(f, "gemm")) ? 1 : (f && !strcmp(f, "smallm")) ? 2 : 0;
  g_knobs.loaded = true;
}
inline bool knob_set(Knob k) {
  if (!g_knobs.loaded) load_knobs();
  return g_knobs.present[k];
}
inline int knob(Knob k, int dflt) { return knob_set(k) ? g_knobs.value[k] : dflt; }

// 2-D map over a row-major e4m3 matrix [rows, K] with row pitch `pitch` bytes;
// boxes of 128 bytes (one swizzle row) x box_rows rows; out-of-range elements read as zero.
int32_t make_map(CUtensorMap* map, uint64_t ptr, int64_t rows, int64_t K, int64_t pitch, int box_rows) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
  cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TG_ERR_ARGS, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return TG_OK;
}

// 2-D map over a row-major bf16 / f16 output [rows, cols] with row pitch `pitch_bytes`, for bulk tensor
// stores of 64-column x 32-row boxes out of 128-byte-swizzled shared memory; stores past the extents are clipped.
int32_t make_out_map(CUtensorMap* map, uint64_t ptr, int64_t rows, int64_t cols, int64_t pitch_bytes, int32_t dtype) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
  cuuint32_t box[2] = {64u, 32u};
  cuuint32_t estr[2] = {1u, 1u};
  const CUtensorMapDataType dt = dtype == TG_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(map, dt, 2, reinterpret_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(TG_ERR_ARGS, "cuTensorMapEncodeTiled (output) failed with CUresult %d", static_cast<int>(r));
  return TG_OK;
}

bool is_out_dtype(int32_t d) { return d == TG_F32 || d == TG_F16 || d == TG_BF16; }
int esize(int32_t d) { return d == TG_F32 ? 4 : (d == TG_F16 || d == TG_BF16) ? 2 : 1; }

// A 2-D e4m3 (or, where the entry point takes it, e5m2) operand with unit inner stride, 16-byte aligned base and pitch.
int32_t check_operand(const TgTensorDesc* t, const char* name, bool allow_e5m2 = false) {
  if (t == nullptr) return fail(TG_ERR_NULL, "%s descriptor is null", name);
  if (t->dtype != TG_F8E4M3 && !(allow_e5m2 && t->dtype == TG_F8E5M2))
    return fail(TG_ERR_DTYPE, "%s must be float8_e4m3fn (dtype code 7)%s, got %d", name,
                allow_e5m2 ? " or float8_e5m2 (5)" : "", t->dtype);
  if (t->ndim != 2) return fail(TG_ERR_ARGS, "%s must be 2-D, got %d-D", name, t->ndim);
  if (t->shape[0] < 0 || t->shape[1] <= 0) return fail(TG_ERR_ARGS, "%s has a bad shape", name);
  if (t->strides[1] != 1 || t->strides[0] < t->shape[1]) return fail(TG_ERR_ARGS, "%s rows must be contiguous", name);
  if (t->shape[0] > 0 && t->ptr == 0) return fail(TG_ERR_NULL, "%s data pointer is null", name);
  if ((t->ptr & 15u) != 0 || (t->strides[0] & 15) != 0)
    return fail(TG_ERR_ALIGN, "%s needs a 16-byte aligned base and row pitch (K %% 16 == 0) for TMA", name);
  if (t->shape[0] > 0x7fffffff || t->shape[1] > 0x7fffffff) return fail(TG_ERR_ARGS, "%s is too large", name);
  return TG_OK;
}

int32_t check_output(const TgTensorDesc* C, int64_t M, int64_t N) {
  if (C == nullptr) return fail(TG_ERR_NULL, "C descriptor is null");
  if (!is_out_dtype(C->dtype)) return fail(TG_ERR_DTYPE, "C must be f32, f16 or bf16, got dtype code %d", C->dtype);
  if (C->ndim != 2 || C->shape[0] != M || C->shape[1] != N)
    return fail(TG_ERR_ARGS, "C must have shape [%lld, %lld]", static_cast<long long>(M), static_cast<long long>(N));
  if (C->strides[1] != 1 || C->strides[0] < N) return fail(TG_ERR_ARGS, "C rows must be contiguous");
  if (M > 0 && N > 0 && C->ptr == 0) return fail(TG_ERR_NULL, "C data pointer is null");
  if ((C->ptr & static_cast<uint64_t>(esize(C->dtype) - 1)) != 0) return fail(TG_ERR_ALIGN, "C is not element aligned");
  return TG_OK;
}

// A bias (f32 / f16 / bf16, or NULL): groups == 0 wants a contiguous [N] vector, groups > 0 a contiguous
// [groups, N] matrix (one bias row per weight of a grouped GEMM).
int32_t check_bias(const TgTensorDesc* bias, int64_t groups, int64_t N) {
  if (bias == nullptr) return TG_OK;
  if (bias->dtype != TG_F32 && bias->dtype != TG_BF16 && bias->dtype != TG_F16)
    return fail(TG_ERR_DTYPE, "bias must be f32, f16 or bf16");
  if (groups == 0) {
    if (bias->ndim != 1 || bias->shape[0] != N || bias->strides[0] != 1)
      return fail(TG_ERR_ARGS, "bias must be a contiguous vector of N elements");
  } else if (bias->ndim != 2 || bias->shape[0] != groups || bias->shape[1] != N || bias->strides[1] != 1 ||
             bias->strides[0] != N) {
    return fail(TG_ERR_ARGS, "bias must be a contiguous [groups, N] matrix");
  }
  if (bias->ptr == 0 && N > 0) return fail(TG_ERR_NULL, "bias data pointer is null");
  return TG_OK;
}

// Process-wide promise (tg_set_static_weights): the B operand of small-M GEMMs is never written by the
// kernel that precedes the GEMM on its stream (weights of a Linear layer), see GemmParams::flags.
int32_t g_static_weights = 0;

// Bound of every device-side wait, microseconds (tg_set_wait_limit_us); 0 = the kernels' 2 s default.
uint32_t g_wait_limit_us = 0;

constexpr uint64_t kWsCounterBytes = 64ull << 10;
constexpr uint64_t kWsPartialBytes = 48ull << 20;

// Split K only when the tiles alone leave most SMs idle.
void choose_splits(int tiles, int num_kb, int num_sms, int64_t tile_floats, int target_ctas, int min_kb, int* splits,
                   int* kbps, int suggested = 0) {
  int s = 1;
  if (suggested > 0) {
    s = suggested;
  } else if (tiles * 2 <= target_ctas && num_kb >= 2 * min_kb) {
    s = target_ctas / tiles;
    const int max_by_k = num_kb / min_kb;
    if (s > max_by_k) s = max_by_k;
  }
  s = knob(kKnobSplits, s);
  if (s < 1) s = 1;
  if (s > num_kb) s = num_kb;
  // the partial tiles of all splits must fit the workspace, whoever chose the split count
  while (s > 1 && static_cast<uint64_t>(tiles) * s * tile_floats * 4 > kWsPartialBytes) --s;
  int per = (num_kb + s - 1) / s;
  s = (num_kb + per - 1) / per;  // every split owns at least one k-block
  (void)num_sms;
  *splits = s;
  *kbps = per;
}

// Small-M decomposition: 128 weight rows per tile and the largest power-of-two number of K splits
// (the cluster size, at most 8) that still fits all CTAs on the GPU at two per SM with at least two
// k-blocks each.  Measured on B200: this beats both fewer splits (too few bytes in flight) and
// narrower tiles.  TILEGYM_B200_SPLITS / TILEGYM_B200_TILE_ROWS override it.
void choose_smallm_config(int64_t N, int num_kb, int num_sms, int mp, int32_t* tile_rows, int32_t* splits,
                          int32_t* kbps) {
  (void)mp;
  const int best_tr = 128;
  const int64_t tiles = (N + best_tr - 1) / best_tr;
  int best_s = 1;
  for (int s = 2; s <= 8; s *= 2) {
    if (tiles * s > 2ll * num_sms || num_kb / s < 2) break;
    best_s = s;
  }
  int s = knob(kKnobSplits, best_s);
  if (s < 1) s = 1;
  if (s > 8) s = 8;
  if (s > num_kb) s = num_kb;
  int per = (num_kb + s - 1) / s;
  s = (num_kb + per - 1) / per;
  int tr = knob(kKnobTileRows, best_tr);
  tr = (tr / 8) * 8;
  if (tr < 16) tr = 16;
  if (tr > 128) tr = 128;
  *tile_rows = tr;
  *splits = s;
  *kbps = per;
}

// K split of the block-scaled 128 x 128 kernel (one persistent CTA per SM), by a cost model in k-block times:
// waves x (k-blocks per unit + tail), where a split unit's tail (partial tile written, fence and counter, the last
// arriver adding s partial tiles) costs about 6 + 1.5 s k-block times; fitted to sweeps of the split count at
// M = 128 and 256 on the DeepSeek-V2 shapes.  Ties go to the smaller split count.
int suggest_splits_blockscaled(int64_t tiles, int num_kb, int num_sms, int min_kb) {
  int best = 1;
  double best_cost = 1e300;
  const int max_s = num_kb / min_kb < 16 ? num_kb / min_kb : 16;
  for (int s = 1; s <= max_s; ++s) {
    const int per = (num_kb + s - 1) / s;
    const int64_t waves = (tiles * s + num_sms - 1) / num_sms;
    const double cost = static_cast<double>(waves) * (per + (s > 1 ? 6.0 + 1.5 * s : 0.0));
    if (cost < best_cost * 0.97) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// K split of the small-M block-scaled kernel (one CTA per SM, the splits of a 128-row weight tile form a cluster
// of at most 8 CTAs).  Only split counts whose CTAs are all resident at once are considered (`resident(s)` =
// clusters of s CTAs the device holds; a second wave would double the time), every CTA gets at least two and at
// most `max_kb` k-blocks (the staged scale table), and among those the cost model picks: set-up + k-blocks per
// CTA + the cluster reduction, in k-block times (0.42 us each, measured).  With more than 32 activation rows a
// CTA that would own more than 16 k-blocks is left to the 128 x 128 tile kernel (measured on N = 5120, K = 12288:
// 24.3 against 21.1 us at M = 128, 17.2 against 20.0 us at M = 16).  TILEGYM_B200_SPLITS forces a count.
// Returns false when nothing qualifies: the 128-row tile kernels then take the problem.
template <typename ResidentFn>
bool choose_bs_smallm_splits(int64_t rows, int64_t tiles, int num_kb, int max_kb, ResidentFn resident, int* splits,
                             int* kbps) {
  int best = 0, best_per = 0;
  double best_cost = 1e300;
  const int forced = knob(kKnobSplits, 0);
  if (forced > 0) {  // taken as asked (rounded to a count in which every split owns a k-block), resident or not
    if (forced > 8) return false;
    const int per = (num_kb + forced - 1) / forced;
    if (per > max_kb) return false;
    *kbps = per;
    *splits = (num_kb + per - 1) / per;
    return true;
  }
  for (int s = 1; s <= 8; ++s) {
    const int per = (num_kb + s - 1) / s;
    if ((num_kb + per - 1) / per != s) continue;  // not a canonical split count
    if (per > max_kb || (s > 1 && per < 2)) continue;
    if (tiles > resident(s)) continue;
    if (rows > 32 && per > 16) continue;  // long k-ranges with many rows: the tile kernel's workspace reduction wins
    const double cost = per + (s > 1 ? 3.0 + 0.5 * s : 0.0);
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
      best_per = per;
    }
  }
  if (best == 0) return false;
  *splits = best;
  *kbps = best_per;
  return true;
}

// Tile width and K split of the single-CTA per-tensor kernel (65 <= M < 512 in practice), by a cost model in
// microseconds fitted to sweeps over (width, split) on the Llama-3.1-8B shapes at M = 96 ... 256:
// waves x (k-blocks per unit x time per k-block + split tail).  A k-block takes 0.19 / 0.24 / 0.42 us for 64 /
// 128 / 256 columns; a split unit's tail (partial tile out, fence and counter, the last arriver adding s partial
// tiles) about 2.5 + (width / 64) (0.5 + 0.9 s) us.  Ties go to the narrower tile and the smaller split count.
void choose_bn_splits_pertensor(int64_t M, int64_t N, int num_kb, int num_sms, int forced_bn, bool may_split, int* bn_out,
                                int* splits_out) {
  const int cand[3] = {64, 128, 256};
  const double t_kb[3] = {0.19, 0.24, 0.42};
  const int64_t tm = (M + 127) / 128;
  double best_cost = 1e300;
  *bn_out = forced_bn > 0 ? forced_bn : 128;
  *splits_out = 1;
  for (int i = 0; i < 3; ++i) {
    if (forced_bn > 0 && cand[i] != forced_bn) continue;
    const int64_t tiles = tm * ((N + cand[i] - 1) / cand[i]);
    const int max_s = !may_split ? 1 : (num_kb / 4 < 8 ? (num_kb / 4 > 1 ? num_kb / 4 : 1) : 8);
    for (int s = 1; s <= max_s; ++s) {
      const int per = (num_kb + s - 1) / s;
      const int64_t waves = (tiles * s + num_sms - 1) / num_sms;
      const double tail = s > 1 ? 2.5 + (cand[i] / 64.0) * (0.5 + 0.9 * s) : 0.0;
      const double cost = static_cast<double>(waves) * (per * t_kb[i] + tail);
      if (cost < best_cost * 0.97) {
        best_cost = cost;
        *bn_out = cand[i];
        *splits_out = s;
      }
    }
  }
}

int choose_bn(int64_t M, int64_t N, int num_sms) {
  // Estimated time = waves x tile width x a per-width efficiency factor
  // (narrow tiles re-read A from shared memory more often per flop).
  const int cand[3] = {256, 128, 64};
  const double penalty[3] = {1.0, 1.42, 2.2};  // measured per-flop cost of 128- and 64-wide tiles vs 256
  int best = 256;
  double best_cost = 1e300;
  const int64_t tm = (M + 128 - 1) / 128;
  for (int i = 0; i < 3; ++i) {
    const int64_t tn = (N + cand[i] - 1) / cand[i];
    const int64_t waves = (tm * tn + num_sms - 1) / num_sms;
    const double cost = static_cast<double>(waves) * cand[i] * penalty[i];
    if (cost < best_cost) {
      best_cost = cost;
      best = cand[i];
    }
  }
  return best;
}

}  // namespace

// Thin exports of the helpers above for entry points that live in other files.
int32_t api_fail(int32_t rc, const char* msg) { return fail(rc, "%s", msg); }
int32_t api_check_operand(const TgTensorDesc* t, const char* name) { return check_operand(t, name); }
int32_t api_check_output(const TgTensorDesc* C, int64_t M, int64_t N) { return check_output(C, M, N); }
int32_t api_make_map(CUtensorMap* map, uint64_t ptr, int64_t rows, int64_t K, int64_t pitch, int box_rows) {
  return make_map(map, ptr, rows, K, pitch, box_rows);
}
uint32_t api_wait_limit_us() { return g_wait_limit_us; }
int32_t api_init_device(int dev, int* num_sms, int32_t** status) {
  int32_t rc = init_device(dev);
  if (rc != TG_OK) return rc;
  *num_sms = g_dev[dev].num_sms;
  *status = g_dev[dev].status;
  return TG_OK;
}
}  // namespace tg

using namespace tg;

extern "C" {

int32_t tg_version(void) { return 100; }

int32_t tg_plan_splits(int32_t kind, int64_t M, int64_t N, int64_t K, int32_t num_sms, int32_t* tile_cols,
                       int32_t* splits) {
  if (tile_cols == nullptr || splits == nullptr) return fail(TG_ERR_NULL, "tile_cols / splits is null");
  if (M <= 0 || N <= 0 || K <= 0 || num_sms <= 0) return fail(TG_ERR_ARGS, "M, N, K and num_sms must be positive");
  const int num_kb = static_cast<int>((K + 127) / 128);
  if (kind == 0) {
    int bn = 128, s = 1;
    choose_bn_splits_pertensor(M, N, num_kb, num_sms, 0, true, &bn, &s);
    *tile_cols = bn;
    *splits = s;
  } else if (kind == 1) {
    const int64_t tiles = ((M + 127) / 128) * ((N + 127) / 128);
    *tile_cols = 128;
    *splits = suggest_splits_blockscaled(tiles, num_kb, num_sms, 4);
  } else {
    return fail(TG_ERR_ARGS, "kind must be 0 (per-tensor, single-CTA tiles) or 1 (block-scaled, 128 x 128 tiles)");
  }
  return TG_OK;
}

void tg_reload_env(void) { load_knobs(); }

uint32_t tg_set_wait_limit_us(uint32_t limit_us) {
  const uint32_t old = g_wait_limit_us;
  g_wait_limit_us = limit_us;
  return old;
}

int32_t tg_set_static_weights(int32_t on) {
  const int32_t old = g_static_weights;
  g_static_weights = on ? 1 : 0;
  return old;
}

const char* tg_last_error_string(void) { return g_err; }

uint64_t tg_fp8_gemm_workspace_bytes(int64_t, int64_t, int64_t) { return kWsCounterBytes + kWsPartialBytes; }

// Shared body of tg_fp8_gemm_pertensor (num_peers == 0) and tg_fp8_gemm_pertensor_allgather (the result
// slab is also stored to peer_ptrs[0 .. num_peers), addresses of the same [M, N] view in peer GPUs' buffers).
static int32_t pertensor_impl(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B, uint64_t scale_a,
                              uint64_t scale_b, float alpha, const TgTensorDesc* bias, float beta, uint64_t workspace,
                              uint64_t workspace_bytes, const uint64_t* peer_ptrs, int32_t num_peers,
                              int32_t device_id, uint64_t stream, bool swiglu = false, uint32_t call_flags = 0) {
  int32_t rc;
  if ((rc = check_operand(A, "A", true)) != TG_OK) return rc;
  if ((rc = check_operand(B, "B", true)) != TG_OK) return rc;
  if (A->dtype != B->dtype) return fail(TG_ERR_DTYPE, "A and B must have the same 8-bit format (both e4m3 or both e5m2)");
  const int32_t fmt_flag = A->dtype == TG_F8E5M2 ? 32 : 0;  // GemmParams::flags bit 5: e5m2 operands
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (B->shape[1] != K) return fail(TG_ERR_ARGS, "A is [M,%lld] but B is [N,%lld]: K must match", (long long)K, (long long)B->shape[1]);
  if (swiglu && N % 128 != 0) return fail(TG_ERR_ARGS, "the SwiGLU epilogue needs N (gate + up rows) to be a multiple of 128, got %lld", (long long)N);
  // SwiGLU: every 64 accumulator columns (32 gate, 32 up) become 32 output columns
  const int64_t N_out = swiglu ? N / 2 : N;
  if ((rc = check_output(C, M, N_out)) != TG_OK) return rc;
  if ((rc = check_bias(bias, 0, N)) != TG_OK) return rc;
  if ((scale_a & 3u) || (scale_b & 3u)) return fail(TG_ERR_ALIGN, "scale pointers must be 4-byte aligned");
  if (M == 0 || N == 0) return TG_OK;

  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  const DeviceState& st = g_dev[device_id];
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.wait_limit_us = g_wait_limit_us;
  p.M = static_cast<int32_t>(M);
  p.N = static_cast<int32_t>(N);
  p.K = static_cast<int32_t>(K);
  p.num_kb = static_cast<int32_t>((K + 127) / 128);
  p.C = reinterpret_cast<void*>(C->ptr);
  p.ldc = C->strides[0];
  p.out_dtype = C->dtype;
  p.scale_a = reinterpret_cast<const float*>(scale_a);
  p.scale_b = reinterpret_cast<const float*>(scale_b);
  p.alpha = alpha;
  p.beta = beta;
  p.bias = bias ? reinterpret_cast<const void*>(bias->ptr) : nullptr;
  p.bias_dtype = bias ? bias->dtype : TG_F32;
  p.status = st.status;
  p.ws_counters = reinterpret_cast<uint32_t*>(workspace);
  p.ws_partial = reinterpret_cast<float*>(workspace + kWsCounterBytes);
  p.flags = fmt_flag;
  const bool have_ws = workspace != 0 && workspace_bytes >= kWsCounterBytes + kWsPartialBytes;

  bool small = M <= 64;
  if (knob_set(kKnobForcePath) && g_knobs.force_path == 1) small = false;

  // The output leaves through bulk tensor stores when it is two bytes wide, not accumulated into, and its
  // rows are 16-byte aligned; the fused all-gather needs that path.
  const bool tma_out_ok = (C->dtype == TG_BF16 || C->dtype == TG_F16) && beta == 0.0f && (C->ptr & 15u) == 0 &&
                          ((C->strides[0] * 2) & 15) == 0;
  // The CTA-pair kernel needs enough 256 x 256 tiles to occupy the GPU: below TILEGYM_B200_PAIR_MIN_TILES (24)
  // of them and M < 512, single-CTA tiles (64 ... 256 columns, optional K split) finish sooner; measured at
  // M = 256: N = K = 4096 11.6 against 12.4 us, N = 4096 K = 14336 25.5 against 29.1 us.
  const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
  const bool pair_fills = M >= 512 || num_peers > 0 || pair_tiles >= knob(kKnobPairMinTiles, 24);
  const bool pair_kernel = swiglu || (M >= 256 && N >= 256 && pair_fills && knob(kKnob2Cta, 1) != 0 &&
                                      !knob_set(kKnobBn) && !knob_set(kKnobSplits));
  if (swiglu) {
    if (!tma_out_ok) return fail(TG_ERR_ARGS, "the SwiGLU epilogue needs a bf16 / f16 output with 16-byte aligned rows");
    small = false;  // only the CTA-pair kernel has this epilogue (it runs any M; rows past M read as zero)
    p.flags |= 4;
  }
  if (num_peers > 0 && !(pair_kernel && tma_out_ok))
    return fail(TG_ERR_ARGS, "the fused all-gather needs M, N >= 256, a bf16 / f16 output with 16-byte aligned rows and beta == 0");

  CUtensorMap tmA, tmB;
  if (small) {
    const int mp = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    p.tiles_m = 1;
    p.tiles_n = static_cast<int32_t>((N + 127) / 128);
    // Default: the K splits of a tile form a thread-block cluster (1, 2, 4 or 8 CTAs) and reduce through
    // distributed shared memory; TILEGYM_B200_SMALLM_WS=1 selects the global-workspace reduction.
    const bool use_ws = knob(kKnobSmallmWs, 0) != 0;
    const bool ws_ok = have_ws;
    // bit 1: launch with programmatic stream serialization (the kernel waits before touching global memory);
    // bit 0: the caller promised static weights, whose loads may then start before that wait
    p.flags = fmt_flag | (knob(kKnobPdl, 1) != 0 ? 2 : 0) |
              (((call_flags & TG_GEMM_STATIC_B) || g_static_weights != 0 || knob(kKnobStaticWeights, 0) != 0) ? 1 : 0);
    choose_smallm_config(N, p.num_kb, st.num_sms, mp, &p.tile_rows, &p.splits, &p.kb_per_split);
    if (use_ws && !ws_ok) {
      p.splits = 1;
      p.kb_per_split = p.num_kb;
    }
    p.tiles_n = static_cast<int32_t>((N + p.tile_rows - 1) / p.tile_rows);
    if (use_ws && (p.tiles_n * 4 > static_cast<int64_t>(kWsCounterBytes / 4) ||
                   static_cast<uint64_t>(p.tiles_n) * p.splits * 128 * mp * 4 > kWsPartialBytes))
      return fail(TG_ERR_ARGS, "N (times the K splits) is too large for the workspace reduction");
    if ((rc = make_map(&tmB, B->ptr, N, K, B->strides[0], p.tile_rows)) != TG_OK) return rc;
    if ((rc = make_map(&tmA, A->ptr, M, K, A->strides[0], mp)) != TG_OK) return rc;
    cudaError_t e = (use_ws || p.splits == 1) ? launch_gemm_smallm(tmB, tmA, p, mp, cs)
                                              : launch_gemm_smallm_cluster(tmB, tmA, p, mp, cs);
    if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "small-M GEMM launch failed: %s", cudaGetErrorString(e));
    return TG_OK;
  }

  // Large problems: CTA-pair kernel (256 x 256 tiles, half the L2 traffic per SM).
  if (pair_kernel) {
    if (knob(kKnobPdl, 1) != 0) p.flags |= 2;  // programmatic dependent launch
    p.tiles_m = static_cast<int32_t>((M + 255) / 256);
    p.tiles_n = static_cast<int32_t>((N + 255) / 256);
    p.splits = 1;
    p.kb_per_split = p.num_kb;
    // tile-rows per raster group: the group's A panels (group_m x 256 x K bytes) stay in L2 while the B panels
    // stream past them; up to ~40 MB of A per group, the tile rows spread evenly over the groups (measured,
    // interleaved A/B runs: M = 8192, N = 28672, K = 8192 2768 TFLOP/s with groups of 16 against 2616 with 12 + 12 + 8;
    // K = 14336 best with two groups of 8)
    int group_m = static_cast<int>((40ll << 20) / (256ll * K));
    if (group_m < 2) group_m = 2;
    if (group_m > p.tiles_m) group_m = p.tiles_m;
    {
      const int groups = (p.tiles_m + group_m - 1) / group_m;
      group_m = (p.tiles_m + groups - 1) / groups;
    }
    group_m = knob(kKnobGroupM, group_m);
    if (group_m < 1) group_m = 1;
    if ((rc = make_map(&tmA, A->ptr, M, K, A->strides[0], 128)) != TG_OK) return rc;
    if ((rc = make_map(&tmB, B->ptr, N, K, B->strides[0], 128)) != TG_OK) return rc;
    // tiles of a partly filled last wave are cut into column slices (TILEGYM_B200_TAIL_DIV overrides: 1, 2, 4)
    int tail_div = pertensor_2cta_tail_div(p.tiles_m * p.tiles_n, st.num_sms);
    tail_div = knob(kKnobTailDiv, tail_div);
    if (tail_div != 2 && tail_div != 4) tail_div = 1;
    if (swiglu && tail_div == 4) tail_div = 2;  // a SwiGLU output box needs 128 accumulator columns
    CUtensorMap tmBt;
    if ((rc = make_map(&tmBt, B->ptr, N, K, B->strides[0], 128 / tail_div)) != TG_OK) return rc;
    CUtensorMap out_maps[8];
    int num_out = 0;
    if (tma_out_ok && (num_peers > 0 || swiglu || knob(kKnobTmaStore, 1) != 0)) {
      if ((rc = make_out_map(&out_maps[num_out++], C->ptr, M, N_out, C->strides[0] * 2, C->dtype)) != TG_OK) return rc;
      for (int i = 0; i < num_peers; ++i)
        if ((rc = make_out_map(&out_maps[num_out++], peer_ptrs[i], M, N, C->strides[0] * 2, C->dtype)) != TG_OK) return rc;
    }
    cudaError_t e2 = launch_gemm_pertensor_2cta(tmA, tmB, tmBt, out_maps, num_out, p, group_m, tail_div, st.num_sms, cs);
    if (e2 != cudaSuccess) return fail(TG_ERR_LAUNCH, "GEMM (CTA pair) launch failed: %s", cudaGetErrorString(e2));
    return TG_OK;
  }

  // programmatic dependent launch: this kernel's set-up overlaps the tail of the previous kernel on the stream
  if (knob(kKnobPdl, 1) != 0) p.flags |= 2;
  const int forced_bn = knob(kKnobBn, 0);
  if (forced_bn != 0 && forced_bn != 256 && forced_bn != 128 && forced_bn != 64)
    return fail(TG_ERR_ARGS, "TILEGYM_B200_BN must be 64, 128 or 256");
  int bn = 128, suggested = 1;
  if (M < 512)
    choose_bn_splits_pertensor(M, N, p.num_kb, st.num_sms, forced_bn, have_ws, &bn, &suggested);
  else
    bn = forced_bn != 0 ? forced_bn : choose_bn(M, N, st.num_sms);  // larger M gets here only with the pair kernel off
  p.tiles_m = static_cast<int32_t>((M + 127) / 128);
  p.tiles_n = static_cast<int32_t>((N + bn - 1) / bn);
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (tiles > 0x3fffffff) return fail(TG_ERR_ARGS, "problem has too many tiles");
  if (have_ws && tiles * 4 <= static_cast<int64_t>(kWsCounterBytes / 4))
    choose_splits(static_cast<int>(tiles), p.num_kb, st.num_sms, 128ll * bn, st.num_sms, 4, &p.splits, &p.kb_per_split,
                  M < 512 ? suggested : 0);
  else {
    p.splits = 1;
    p.kb_per_split = p.num_kb;
  }
  if ((rc = make_map(&tmA, A->ptr, M, K, A->strides[0], 128)) != TG_OK) return rc;
  if ((rc = make_map(&tmB, B->ptr, N, K, B->strides[0], bn)) != TG_OK) return rc;
  cudaError_t e = launch_gemm_pertensor(tmA, tmB, p, bn, st.num_sms, cs);
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "GEMM launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

int32_t tg_fp8_gemm_pertensor(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B, uint64_t scale_a,
                              uint64_t scale_b, float alpha, const TgTensorDesc* bias, float beta, uint64_t workspace,
                              uint64_t workspace_bytes, uint32_t flags, int32_t device_id, uint64_t stream) {
  if (flags & ~TG_GEMM_STATIC_B) return fail(TG_ERR_ARGS, "unknown flag bits 0x%x", flags & ~TG_GEMM_STATIC_B);
  return pertensor_impl(C, A, B, scale_a, scale_b, alpha, bias, beta, workspace, workspace_bytes, nullptr, 0,
                        device_id, stream, false, flags);
}

int32_t tg_fp8_gemm_pertensor_allgather(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                        uint64_t scale_a, uint64_t scale_b, float alpha, const TgTensorDesc* bias,
                                        const uint64_t* peer_ptrs, int32_t num_peers, int32_t device_id,
                                        uint64_t stream) {
  if (num_peers < 0 || num_peers > 7) return fail(TG_ERR_ARGS, "num_peers must be 0..7, got %d", num_peers);
  if (num_peers > 0 && peer_ptrs == nullptr) return fail(TG_ERR_NULL, "peer_ptrs is null");
  for (int i = 0; i < num_peers; ++i) {
    if (peer_ptrs[i] == 0) return fail(TG_ERR_NULL, "peer pointer %d is null", i);
    if (peer_ptrs[i] & 15u) return fail(TG_ERR_ALIGN, "peer pointer %d is not 16-byte aligned", i);
  }
  return pertensor_impl(C, A, B, scale_a, scale_b, alpha, bias, 0.0f, 0, 0, peer_ptrs, num_peers, device_id, stream);
}

// ncclAllGather of the NCCL library the process already uses (torch's, or whatever the caller linked), resolved at
// run time so that this library has no link-time dependency on NCCL.
typedef int (*NcclAllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
static NcclAllGatherFn resolve_nccl_allgather() {
  static NcclAllGatherFn fn = nullptr;
  static bool tried = false;
  if (tried) return fn;
  tried = true;
  void* sym = dlsym(RTLD_DEFAULT, "ncclAllGather");
  if (sym == nullptr) {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // already loaded under that name (e.g. by torch)?
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h != nullptr) sym = dlsym(h, "ncclAllGather");
  }
  fn = reinterpret_cast<NcclAllGatherFn>(sym);
  return fn;
}

int32_t tg_shard_gemm_allgather(const TgTensorDesc* C_all, const TgTensorDesc* A, const TgTensorDesc* B_shard,
                                uint64_t scale_a, uint64_t scale_b, float alpha, const TgTensorDesc* bias_shard,
                                int32_t rank, int32_t world, uint64_t comm, uint64_t workspace,
                                uint64_t workspace_bytes, int32_t device_id, uint64_t stream) {
  if (C_all == nullptr || A == nullptr || B_shard == nullptr) return fail(TG_ERR_NULL, "a descriptor is null");
  if (world < 1 || rank < 0 || rank >= world) return fail(TG_ERR_ARGS, "rank %d of %d is out of range", rank, world);
  if (C_all->ndim != 3 || C_all->shape[0] != world) return fail(TG_ERR_ARGS, "C_all must be [world, M, n]");
  if (!is_out_dtype(C_all->dtype)) return fail(TG_ERR_DTYPE, "C_all must be f32, f16 or bf16");
  const int64_t M = C_all->shape[1], n = C_all->shape[2];
  if (M > 0 && n > 0 && (C_all->strides[2] != 1 || C_all->strides[1] != n || C_all->strides[0] != M * n))
    return fail(TG_ERR_ARGS, "C_all must be contiguous (NCCL gathers contiguous slabs)");
  if (world > 1 && comm == 0) return fail(TG_ERR_NULL, "comm (ncclComm_t) is null");
  TgTensorDesc slab;
  memset(&slab, 0, sizeof(slab));
  slab.ptr = C_all->ptr + static_cast<uint64_t>(rank) * M * n * esize(C_all->dtype);
  slab.ndim = 2;
  slab.shape[0] = M;
  slab.shape[1] = n;
  slab.strides[0] = n;
  slab.strides[1] = 1;
  slab.dtype = C_all->dtype;
  int32_t rc = pertensor_impl(&slab, A, B_shard, scale_a, scale_b, alpha, bias_shard, 0.0f, workspace, workspace_bytes,
                              nullptr, 0, device_id, stream);
  if (rc != TG_OK || world == 1 || M == 0 || n == 0) return rc;
  NcclAllGatherFn gather = resolve_nccl_allgather();
  if (gather == nullptr) return fail(TG_ERR_DEVICE, "ncclAllGather not found: no libnccl.so.2 is loaded or loadable in this process");
  const int nccl_dtype = C_all->dtype == TG_BF16 ? 9 : (C_all->dtype == TG_F16 ? 6 : 7);  // ncclBfloat16 / Float16 / Float32
  DeviceGuard guard(device_id);
  const int r = gather(reinterpret_cast<const void*>(slab.ptr), reinterpret_cast<void*>(C_all->ptr),
                       static_cast<size_t>(M) * static_cast<size_t>(n), nccl_dtype, reinterpret_cast<void*>(comm),
                       reinterpret_cast<cudaStream_t>(stream));
  if (r != 0) return fail(TG_ERR_LAUNCH, "ncclAllGather failed with ncclResult_t %d", r);
  return TG_OK;
}

int32_t tg_fp8_gemm_pertensor_swiglu(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                     uint64_t scale_a, uint64_t scale_b, float alpha, const TgTensorDesc* bias,
                                     int32_t device_id, uint64_t stream) {
  return pertensor_impl(C, A, B, scale_a, scale_b, alpha, bias, 0.0f, 0, 0, nullptr, 0, device_id, stream, true);
}

// Dense bf16 / f16 GEMM on the CTA-pair kernel (tcgen05 kind::f16): the unquantised path of `matmul`.
int32_t tg_gemm_dense16(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B, float alpha,
                        const TgTensorDesc* bias, float beta, int32_t device_id, uint64_t stream) {
  int32_t rc;
  if (A == nullptr || B == nullptr) return fail(TG_ERR_NULL, "a descriptor is null");
  if ((A->dtype != TG_BF16 && A->dtype != TG_F16) || B->dtype != A->dtype)
    return fail(TG_ERR_DTYPE, "A and B must both be bf16 or both f16");
  if (A->ndim != 2 || B->ndim != 2) return fail(TG_ERR_ARGS, "A and B must be 2-D");
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (K <= 0 || B->shape[1] != K) return fail(TG_ERR_ARGS, "A is [M,%lld] but B is [N,%lld]: K must match", (long long)K, (long long)B->shape[1]);
  if (A->strides[1] != 1 || B->strides[1] != 1 || A->strides[0] < K || B->strides[0] < K)
    return fail(TG_ERR_ARGS, "A and B rows must be contiguous");
  if ((M > 0 && A->ptr == 0) || (N > 0 && B->ptr == 0)) return fail(TG_ERR_NULL, "data pointer is null");
  if ((A->ptr & 15u) || (B->ptr & 15u) || ((A->strides[0] * 2) & 15) || ((B->strides[0] * 2) & 15))
    return fail(TG_ERR_ALIGN, "A and B need 16-byte aligned bases and row pitches (K %% 8 == 0) for TMA");
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return fail(TG_ERR_ARGS, "problem is too large");
  if ((rc = check_output(C, M, N)) != TG_OK) return rc;
  if ((rc = check_bias(bias, 0, N)) != TG_OK) return rc;
  if (M == 0 || N == 0) return TG_OK;

  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  const DeviceState& st = g_dev[device_id];
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.wait_limit_us = g_wait_limit_us;
  p.M = static_cast<int32_t>(M);
  p.N = static_cast<int32_t>(N);
  p.K = static_cast<int32_t>(K);
  p.num_kb = static_cast<int32_t>((K + 63) / 64);  // a k-block is one 128-byte row of 64 elements
  p.tiles_m = static_cast<int32_t>((M + 255) / 256);
  p.tiles_n = static_cast<int32_t>((N + 255) / 256);
  p.C = reinterpret_cast<void*>(C->ptr);
  p.ldc = C->strides[0];
  p.out_dtype = C->dtype;
  p.alpha = alpha;
  p.beta = beta;
  p.bias = bias ? reinterpret_cast<const void*>(bias->ptr) : nullptr;
  p.bias_dtype = bias ? bias->dtype : TG_F32;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.status = st.status;
  p.flags = ((A->dtype == TG_BF16) ? 8 : 16) | (knob(kKnobPdl, 1) != 0 ? 2 : 0);

  auto map16 = [&](CUtensorMap* map, const TgTensorDesc* t, int64_t rows, int box_rows) -> int32_t {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(t->strides[0] * 2)};
    cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = g_encode(map, t->dtype == TG_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                          reinterpret_cast<void*>(t->ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TG_OK : fail(TG_ERR_ARGS, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  };
  int group_m = static_cast<int>((24ll << 20) / (512ll * K));
  if (group_m < 2) group_m = 2;
  if (group_m > p.tiles_m) group_m = p.tiles_m;
  int tail_div = pertensor_2cta_tail_div(p.tiles_m * p.tiles_n, st.num_sms);
  if (tail_div != 2 && tail_div != 4) tail_div = 1;
  CUtensorMap tmA, tmB, tmBt;
  if ((rc = map16(&tmA, A, M, 128)) != TG_OK) return rc;
  if ((rc = map16(&tmB, B, N, 128)) != TG_OK) return rc;
  if ((rc = map16(&tmBt, B, N, 128 / tail_div)) != TG_OK) return rc;
  const bool tma_out_ok = (C->dtype == TG_BF16 || C->dtype == TG_F16) && beta == 0.0f && (C->ptr & 15u) == 0 &&
                          ((C->strides[0] * 2) & 15) == 0;
  CUtensorMap out_maps[8];
  int num_out = 0;
  if (tma_out_ok && (rc = make_out_map(&out_maps[num_out++], C->ptr, M, N, C->strides[0] * 2, C->dtype)) != TG_OK) return rc;
  cudaError_t e = launch_gemm_pertensor_2cta(tmA, tmB, tmBt, out_maps, num_out, p, group_m, tail_div, st.num_sms, cs);
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "dense GEMM launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

// Tile order of the grouped kernel (GemmParams flags bit 6).  With few rows per group (a mixture-of-experts layer:
// 3-4 row tiles per expert) the column tiles of one row tile run next to each other, so a group's activations and
// weights are used within one short window and each is read from HBM once; with many rows per group the row tiles
// vary fastest and the CTAs running together share a few weight panels.  TILEGYM_B200_GROUP_ORDER=1 / 2 forces
// row-fastest / column-fastest.
static int grouped_order_flag(int64_t M, int64_t G) {
  const int forced = knob(kKnobGroupOrder, 0);
  if (forced == 1) return 0;
  if (forced == 2) return 64;
  return (G > 0 && M / G < 512) ? 64 : 0;  // measured: 64 groups x 384 rows -8 % / -5 % (K = 2048 / 1536), 8 x 512 rows +1 %
}

int32_t tg_fp8_gemm_blockscaled_grouped(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                        const TgTensorDesc* As, const TgTensorDesc* Bs, uint64_t m_indptr,
                                        int32_t block_n, int32_t block_k, const TgTensorDesc* bias, float beta,
                                        uint64_t row_scale, int32_t device_id, uint64_t stream) {
  int32_t rc;
  if ((rc = check_operand(A, "A")) != TG_OK) return rc;
  if (B == nullptr || As == nullptr || Bs == nullptr) return fail(TG_ERR_NULL, "a descriptor is null");
  if (B->dtype != TG_F8E4M3) return fail(TG_ERR_DTYPE, "B must be float8_e4m3fn (dtype code 7), got %d", B->dtype);
  if (block_n != 128 || block_k != 128)
    return fail(TG_ERR_ARGS, "only block_size [128, 128] is implemented, got [%d, %d]", block_n, block_k);
  if (B->ndim != 3) return fail(TG_ERR_ARGS, "B must be [groups, N, K], got %d-D", B->ndim);
  const int64_t M = A->shape[0], K = A->shape[1], G = B->shape[0], N = B->shape[1];
  if (G <= 0 || N <= 0 || B->shape[2] != K) return fail(TG_ERR_ARGS, "B must be [groups >= 1, N >= 1, K = %lld]", (long long)K);
  if (B->strides[2] != 1 || B->strides[1] != K || B->strides[0] != N * K) return fail(TG_ERR_ARGS, "B must be contiguous");
  if (B->ptr == 0) return fail(TG_ERR_NULL, "B data pointer is null");
  if ((B->ptr & 15u) != 0 || (K & 15) != 0) return fail(TG_ERR_ALIGN, "B needs a 16-byte aligned base and K %% 16 == 0 for TMA");
  if (G * N > 0x7fffffff || G > 0x7fffff) return fail(TG_ERR_ARGS, "B is too large");
  if ((rc = check_output(C, M, N)) != TG_OK) return rc;
  const int64_t KB = (K + 127) / 128, NB = (N + 127) / 128;
  if (As->dtype != TG_F32 || Bs->dtype != TG_F32) return fail(TG_ERR_DTYPE, "As and Bs must be f32");
  if (As->ndim != 2 || As->shape[0] != M || As->shape[1] != KB || As->strides[1] != 1 || As->strides[0] < KB)
    return fail(TG_ERR_ARGS, "As must be [M, ceil(K/128)] = [%lld, %lld] with contiguous rows", (long long)M, (long long)KB);
  if (Bs->ndim != 3 || Bs->shape[0] != G || Bs->shape[1] != NB || Bs->shape[2] != KB || Bs->strides[2] != 1 ||
      Bs->strides[1] != KB || Bs->strides[0] != NB * KB)
    return fail(TG_ERR_ARGS, "Bs must be contiguous [groups, ceil(N/128), ceil(K/128)] = [%lld, %lld, %lld]", (long long)G,
                (long long)NB, (long long)KB);
  if ((M > 0 && As->ptr == 0) || Bs->ptr == 0) return fail(TG_ERR_NULL, "scale data pointer is null");
  if ((As->ptr & 3u) || (Bs->ptr & 3u)) return fail(TG_ERR_ALIGN, "scale pointers must be 4-byte aligned");
  if (m_indptr == 0) return fail(TG_ERR_NULL, "m_indptr is null");
  if (m_indptr & 3u) return fail(TG_ERR_ALIGN, "m_indptr must be 4-byte aligned");
  if (row_scale & 3u) return fail(TG_ERR_ALIGN, "row_scale must be 4-byte aligned");
  if ((rc = check_bias(bias, G, N)) != TG_OK) return rc;
  if (M == 0) return TG_OK;

  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  const DeviceState& st = g_dev[device_id];
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.wait_limit_us = g_wait_limit_us;
  p.M = static_cast<int32_t>(M);
  p.N = static_cast<int32_t>(N);
  p.K = static_cast<int32_t>(K);
  p.num_kb = static_cast<int32_t>(KB);
  p.tiles_n = static_cast<int32_t>((N + 255) / 256);
  p.C = reinterpret_cast<void*>(C->ptr);
  p.ldc = C->strides[0];
  p.out_dtype = C->dtype;
  p.alpha = 1.0f;
  p.beta = beta;
  p.bias = bias ? reinterpret_cast<const void*>(bias->ptr) : nullptr;
  p.bias_dtype = bias ? bias->dtype : TG_F32;
  p.As = reinterpret_cast<const float*>(As->ptr);
  p.Bs = reinterpret_cast<const float*>(Bs->ptr);
  p.ldas = As->strides[0];
  p.ldbs = KB;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.status = st.status;
  if (knob(kKnobPdl, 1) != 0) p.flags |= 2;  // programmatic dependent launch
  p.flags |= grouped_order_flag(M, G);
  p.m_indptr = reinterpret_cast<const int32_t*>(m_indptr);
  p.row_scale = reinterpret_cast<const float*>(row_scale);
  p.num_groups = static_cast<int32_t>(G);
  // Few rows per group (a mixture-of-experts layer at decode sizes): the swap-AB small-M kernel in its grouped form
  // streams each group's weights once for a 32- or 64-row tile instead of a 128-row one, of which most would be
  // other groups' rows.  TILEGYM_B200_GROUPED_SMALLM=0 switches it off, 32 / 64 force the tile height.
  {
    const int forced = knob(kKnobGroupedSmallm, -1);
    int mp = 0;
    if (forced == 32 || forced == 64) mp = forced;
    else if (forced != 0) mp = M <= 24 * G ? 32 : (M <= 64 * G ? 64 : 0);  // measured cross-overs (64 groups, K = 2048 / 1536)
    if (mp != 0 && beta == 0.0f && KB <= blockscaled_smallm_max_kb_per_cta()) {
      // every group adds at most one partly filled tile, and there are never more tiles than rows
      const int64_t mbound = std::min<int64_t>((M + mp - 1) / mp + G, M);
      if (mbound * NB <= 0x3fffffff) {
        p.tiles_m = 1;
        p.tiles_n = static_cast<int32_t>(NB);
        p.mtile_bound = static_cast<int32_t>(mbound);
        CUtensorMap tmW, tmX;
        if ((rc = make_map(&tmW, B->ptr, G * N, K, K, 128)) != TG_OK) return rc;  // B viewed as [G * N, K]
        if ((rc = make_map(&tmX, A->ptr, M, K, A->strides[0], mp)) != TG_OK) return rc;
        cudaError_t e0 = launch_gemm_blockscaled_smallm_grouped(tmW, tmX, p, mp, cs);
        if (e0 != cudaSuccess)
          return fail(TG_ERR_LAUNCH, "grouped block-scaled GEMM (small groups) launch failed: %s", cudaGetErrorString(e0));
        return TG_OK;
      }
    }
  }
  // every group adds at most one partly filled 128-row tile to the ceil(M / 128) a dense problem would have
  const int64_t bound = (M + 127) / 128 + G;
  if (bound * p.tiles_n > 0x3fffffff) return fail(TG_ERR_ARGS, "problem has too many tiles");
  p.mtile_bound = static_cast<int32_t>(bound);
  CUtensorMap tmA, tmB, tmC;
  if ((rc = make_map(&tmA, A->ptr, M, K, A->strides[0], 128)) != TG_OK) return rc;
  if ((rc = make_map(&tmB, B->ptr, G * N, K, K, 256)) != TG_OK) return rc;  // B viewed as [G * N, K]
  const bool tma_out = (C->dtype == TG_BF16 || C->dtype == TG_F16) && beta == 0.0f && (C->ptr & 15u) == 0 &&
                       ((C->strides[0] * 2) & 15) == 0 && knob(kKnobTmaStore, 1) != 0;
  if (tma_out && (rc = make_out_map(&tmC, C->ptr, M, N, C->strides[0] * 2, C->dtype)) != TG_OK) return rc;
  cudaError_t e = launch_gemm_blockscaled_grouped(tmA, tmB, tma_out ? &tmC : nullptr, p, st.num_sms, cs);
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "grouped block-scaled GEMM launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

// First GEMM of a mixture-of-experts layer with SiLU * mul and the e4m3 quantisation in its epilogue.
int32_t tg_fp8_gemm_blockscaled_grouped_swiglu(const TgTensorDesc* Y, const TgTensorDesc* Ys, const TgTensorDesc* A,
                                               const TgTensorDesc* B, const TgTensorDesc* As, const TgTensorDesc* Bs,
                                               uint64_t m_indptr, int32_t round_dtype, int32_t quant_mode,
                                               int32_t device_id, uint64_t stream) {
  int32_t rc;
  if ((rc = check_operand(A, "A")) != TG_OK) return rc;
  if (Y == nullptr || Ys == nullptr || B == nullptr || As == nullptr || Bs == nullptr) return fail(TG_ERR_NULL, "a descriptor is null");
  if (B->dtype != TG_F8E4M3 || Y->dtype != TG_F8E4M3) return fail(TG_ERR_DTYPE, "B and Y must be float8_e4m3fn");
  if (round_dtype != TG_BF16 && round_dtype != TG_F16) return fail(TG_ERR_DTYPE, "round_dtype must be bf16 or f16");
  if (quant_mode != 0 && quant_mode != 1) return fail(TG_ERR_ARGS, "quant_mode must be 0 (scale 1) or 1 (amax / 448 per 128 outputs)");
  if (B->ndim != 3) return fail(TG_ERR_ARGS, "B must be [groups, N, K], got %d-D", B->ndim);
  const int64_t M = A->shape[0], K = A->shape[1], G = B->shape[0], N = B->shape[1];
  if (G <= 0 || N <= 0 || B->shape[2] != K) return fail(TG_ERR_ARGS, "B must be [groups >= 1, N >= 1, K = %lld]", (long long)K);
  if (N % 256 != 0) return fail(TG_ERR_ARGS, "N (gate + up rows, alternating in blocks of 128) must be a multiple of 256, got %lld", (long long)N);
  if (B->strides[2] != 1 || B->strides[1] != K || B->strides[0] != N * K) return fail(TG_ERR_ARGS, "B must be contiguous");
  if (B->ptr == 0) return fail(TG_ERR_NULL, "B data pointer is null");
  if ((B->ptr & 15u) != 0 || (K & 15) != 0) return fail(TG_ERR_ALIGN, "B needs a 16-byte aligned base and K %% 16 == 0 for TMA");
  if (G * N > 0x7fffffff || G > 0x7fffff) return fail(TG_ERR_ARGS, "B is too large");
  const int64_t KB = (K + 127) / 128, NB = N / 128, I = N / 2;
  if (Y->ndim != 2 || Y->shape[0] != M || Y->shape[1] != I || Y->strides[1] != 1 || Y->strides[0] != I)
    return fail(TG_ERR_ARGS, "Y must be a contiguous [M, N / 2] matrix");
  if (Ys->dtype != TG_F32 || Ys->ndim != 2 || Ys->shape[0] != M || Ys->shape[1] != I / 128 || Ys->strides[1] != 1 ||
      Ys->strides[0] != I / 128)
    return fail(TG_ERR_ARGS, "Ys must be a contiguous f32 [M, N / 256] matrix");
  if (As->dtype != TG_F32 || Bs->dtype != TG_F32) return fail(TG_ERR_DTYPE, "As and Bs must be f32");
  if (As->ndim != 2 || As->shape[0] != M || As->shape[1] != KB || As->strides[1] != 1 || As->strides[0] < KB)
    return fail(TG_ERR_ARGS, "As must be [M, ceil(K/128)] with contiguous rows");
  if (Bs->ndim != 3 || Bs->shape[0] != G || Bs->shape[1] != NB || Bs->shape[2] != KB || Bs->strides[2] != 1 ||
      Bs->strides[1] != KB || Bs->strides[0] != NB * KB)
    return fail(TG_ERR_ARGS, "Bs must be contiguous [groups, N / 128, ceil(K/128)]");
  if (m_indptr == 0) return fail(TG_ERR_NULL, "m_indptr is null");
  if (m_indptr & 3u) return fail(TG_ERR_ALIGN, "m_indptr must be 4-byte aligned");
  if (M == 0) return TG_OK;
  if (Y->ptr == 0 || Ys->ptr == 0 || As->ptr == 0 || Bs->ptr == 0) return fail(TG_ERR_NULL, "data pointer is null");
  if ((Y->ptr & 15u) || (Ys->ptr & 3u) || (As->ptr & 3u) || (Bs->ptr & 3u)) return fail(TG_ERR_ALIGN, "Y must be 16-byte, scales 4-byte aligned");

  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  const DeviceState& st = g_dev[device_id];
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.wait_limit_us = g_wait_limit_us;
  p.M = static_cast<int32_t>(M);
  p.N = static_cast<int32_t>(N);
  p.K = static_cast<int32_t>(K);
  p.num_kb = static_cast<int32_t>(KB);
  p.tiles_n = static_cast<int32_t>(N / 256);
  p.C = reinterpret_cast<void*>(Y->ptr);
  p.ldc = I;
  p.out_dtype = round_dtype;
  p.alpha = 1.0f;
  p.As = reinterpret_cast<const float*>(As->ptr);
  p.Bs = reinterpret_cast<const float*>(Bs->ptr);
  p.ldas = As->strides[0];
  p.ldbs = KB;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.status = st.status;
  if (knob(kKnobPdl, 1) != 0) p.flags |= 2;
  p.flags |= grouped_order_flag(M, G);
  p.m_indptr = reinterpret_cast<const int32_t*>(m_indptr);
  p.num_groups = static_cast<int32_t>(G);
  p.y_scale = reinterpret_cast<float*>(Ys->ptr);
  p.quant_mode = quant_mode;
  const int64_t bound = (M + 127) / 128 + G;
  if (bound * p.tiles_n > 0x3fffffff) return fail(TG_ERR_ARGS, "problem has too many tiles");
  p.mtile_bound = static_cast<int32_t>(bound);
  CUtensorMap tmA, tmB;
  if ((rc = make_map(&tmA, A->ptr, M, K, A->strides[0], 128)) != TG_OK) return rc;
  if ((rc = make_map(&tmB, B->ptr, G * N, K, K, 256)) != TG_OK) return rc;
  cudaError_t e = launch_gemm_blockscaled_grouped_swiglu(tmA, tmB, p, st.num_sms, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "grouped block-scaled GEMM (SiLU * mul epilogue) launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

int32_t tg_fp8_gemm_blockscaled(const TgTensorDesc* C, const TgTensorDesc* A, const TgTensorDesc* B,
                                const TgTensorDesc* As, const TgTensorDesc* Bs, int32_t block_n, int32_t block_k,
                                const TgTensorDesc* bias, float beta, uint64_t workspace, uint64_t workspace_bytes,
                                int32_t device_id, uint64_t stream) {
  int32_t rc;
  if ((rc = check_operand(A, "A")) != TG_OK) return rc;
  if ((rc = check_operand(B, "B")) != TG_OK) return rc;
  if (As == nullptr || Bs == nullptr) return fail(TG_ERR_NULL, "scale descriptor is null");
  if (block_n != 128 || block_k != 128)
    return fail(TG_ERR_ARGS, "only block_size [128, 128] is implemented (the tile is locked to the quantisation block), got [%d, %d]", block_n, block_k);
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (B->shape[1] != K) return fail(TG_ERR_ARGS, "A is [M,%lld] but B is [N,%lld]: K must match", (long long)K, (long long)B->shape[1]);
  if ((rc = check_output(C, M, N)) != TG_OK) return rc;
  const int64_t KB = (K + 127) / 128, NB = (N + 127) / 128;
  if (As->dtype != TG_F32 || Bs->dtype != TG_F32) return fail(TG_ERR_DTYPE, "As and Bs must be f32");
  if (As->ndim != 2 || As->shape[0] != M || As->shape[1] != KB || As->strides[1] != 1 || As->strides[0] < KB)
    return fail(TG_ERR_ARGS, "As must be [M, ceil(K/128)] = [%lld, %lld] with contiguous rows", (long long)M, (long long)KB);
  if (Bs->ndim != 2 || Bs->shape[0] != NB || Bs->shape[1] != KB || Bs->strides[1] != 1 || Bs->strides[0] < KB)
    return fail(TG_ERR_ARGS, "Bs must be [ceil(N/128), ceil(K/128)] = [%lld, %lld] with contiguous rows", (long long)NB, (long long)KB);
  if ((M > 0 && As->ptr == 0) || (N > 0 && Bs->ptr == 0)) return fail(TG_ERR_NULL, "scale data pointer is null");
  if ((As->ptr & 3u) || (Bs->ptr & 3u)) return fail(TG_ERR_ALIGN, "scale pointers must be 4-byte aligned");
  if ((rc = check_bias(bias, 0, N)) != TG_OK) return rc;
  if (M == 0 || N == 0) return TG_OK;

  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  const DeviceState& st = g_dev[device_id];
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.wait_limit_us = g_wait_limit_us;
  p.M = static_cast<int32_t>(M);
  p.N = static_cast<int32_t>(N);
  p.K = static_cast<int32_t>(K);
  p.num_kb = static_cast<int32_t>(KB);
  p.tiles_m = static_cast<int32_t>((M + 127) / 128);
  p.tiles_n = static_cast<int32_t>(NB);
  p.C = reinterpret_cast<void*>(C->ptr);
  p.ldc = C->strides[0];
  p.out_dtype = C->dtype;
  p.alpha = 1.0f;
  p.beta = beta;
  p.bias = bias ? reinterpret_cast<const void*>(bias->ptr) : nullptr;
  p.bias_dtype = bias ? bias->dtype : TG_F32;
  p.As = reinterpret_cast<const float*>(As->ptr);
  p.Bs = reinterpret_cast<const float*>(Bs->ptr);
  p.ldas = As->strides[0];
  p.ldbs = Bs->strides[0];
  p.status = st.status;
  if (knob(kKnobPdl, 1) != 0) p.flags |= 2;  // programmatic dependent launch
  p.ws_counters = reinterpret_cast<uint32_t*>(workspace);
  p.ws_partial = reinterpret_cast<float*>(workspace + kWsCounterBytes);
  const bool have_ws = workspace != 0 && workspace_bytes >= kWsCounterBytes + kWsPartialBytes;
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (tiles > 0x3fffffff) return fail(TG_ERR_ARGS, "problem has too many tiles");
  // Small M (M <= 128, no beta): the swap-AB kernel (weights on the MMA M axis, K splits reduced inside a
  // cluster); TILEGYM_B200_BS_SMALLM=0 switches it off.
  // M <= 64, a short K and at least as many weight tiles as SMs (e.g. N = 24576, K = 1536): one short CTA per
  // (row tile, weight tile), two per SM, no K split - the launch shape of the grouped small-M kernel with one group.
  if (M <= 64 && beta == 0.0f && knob(kKnobBsSmallm, 1) != 0 && p.num_kb <= blockscaled_smallm_max_kb_per_cta() &&
      NB >= st.num_sms && knob(kKnobGroupedSmallm, -1) != 0) {
    const int mp = M <= 32 ? 32 : 64;
    p.tiles_m = 1;
    p.tiles_n = static_cast<int32_t>(NB);
    p.splits = 1;
    p.kb_per_split = p.num_kb;
    p.num_groups = 1;
    p.m_indptr = nullptr;
    p.mtile_bound = static_cast<int32_t>((M + mp - 1) / mp);
    if (knob(kKnobPdl, 1) != 0) p.flags |= 2;
    CUtensorMap tmW, tmX;
    if ((rc = make_map(&tmW, B->ptr, N, K, B->strides[0], 128)) != TG_OK) return rc;
    if ((rc = make_map(&tmX, A->ptr, M, K, A->strides[0], mp)) != TG_OK) return rc;
    cudaError_t e0 = launch_gemm_blockscaled_smallm_grouped(tmW, tmX, p, mp, cs);
    if (e0 != cudaSuccess) return fail(TG_ERR_LAUNCH, "block-scaled GEMM (small M, many tiles) launch failed: %s", cudaGetErrorString(e0));
    return TG_OK;
  }
  if (M <= 128 && beta == 0.0f && knob(kKnobBsSmallm, 1) != 0) {
    int s = 0, per = 0;
    const int mp = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
    const int sms = st.num_sms;
    if (choose_bs_smallm_splits(M, NB, p.num_kb, blockscaled_smallm_max_kb_per_cta(),
                                [mp, sms](int sp) { return blockscaled_smallm_resident_clusters(mp, sp, sms); }, &s, &per)) {
      p.tiles_m = 1;
      p.tiles_n = static_cast<int32_t>(NB);
      p.splits = s;
      p.kb_per_split = per;
      if (g_static_weights != 0 || knob(kKnobStaticWeights, 0) != 0) p.flags |= 1;
      CUtensorMap tmW, tmX;
      if ((rc = make_map(&tmW, B->ptr, N, K, B->strides[0], 128)) != TG_OK) return rc;
      if ((rc = make_map(&tmX, A->ptr, M, K, A->strides[0], mp)) != TG_OK) return rc;
      cudaError_t e0 = launch_gemm_blockscaled_smallm(tmW, tmX, p, mp, cs);
      if (e0 != cudaSuccess)
        return fail(TG_ERR_LAUNCH, "block-scaled GEMM (small M) launch failed: %s", cudaGetErrorString(e0));
      return TG_OK;
    }
  }
  if (have_ws && tiles * 16 <= static_cast<int64_t>(kWsCounterBytes / 4)) {
    // a problem that fills half a wave of 128 x 256 tiles goes to the wide kernel, which has no K split
    const bool wide_unsplit = static_cast<int64_t>(p.tiles_m) * ((N + 255) / 256) >=
                                  knob(kKnobBsWideMin, (st.num_sms + 1) / 2) &&
                              knob(kKnobBsWide, 1) != 0;
    choose_splits(static_cast<int>(tiles), p.num_kb, st.num_sms, 128ll * 128, st.num_sms, 4, &p.splits, &p.kb_per_split,
                  wide_unsplit ? 1 : suggest_splits_blockscaled(tiles, p.num_kb, st.num_sms, 4));
  } else {
    p.splits = 1;
    p.kb_per_split = p.num_kb;
  }
  CUtensorMap tmA, tmB;
  if ((rc = make_map(&tmA, A->ptr, M, K, A->strides[0], 128)) != TG_OK) return rc;
  if ((rc = make_map(&tmB, B->ptr, N, K, B->strides[0], 128)) != TG_OK) return rc;
  // Problems with at least half a wave of 128 x 256 tiles (and no K split) take the wide-tile kernel (a third
  // less shared-memory traffic per flop than 128 x 128 tiles); TILEGYM_B200_BS_WIDE=0 keeps them on the
  // 128 x 128 kernel.
  const int64_t wide_tiles = static_cast<int64_t>(p.tiles_m) * ((N + 255) / 256);
  // two-byte outputs with 16-byte aligned rows leave through shared memory and bulk tensor stores
  CUtensorMap tmC;
  const bool tma_out = (C->dtype == TG_BF16 || C->dtype == TG_F16) && beta == 0.0f && (C->ptr & 15u) == 0 &&
                       ((C->strides[0] * 2) & 15) == 0 && knob(kKnobTmaStore, 1) != 0;
  if (tma_out && (rc = make_out_map(&tmC, C->ptr, M, N, C->strides[0] * 2, C->dtype)) != TG_OK) return rc;
  // (measured: from half a wave of wide tiles on, the wide kernel also streams a small-M problem faster)
  if (p.splits == 1 && wide_tiles >= knob(kKnobBsWideMin, (st.num_sms + 1) / 2) &&
      knob(kKnobBsWide, 1) != 0) {
    if ((rc = make_map(&tmB, B->ptr, N, K, B->strides[0], 256)) != TG_OK) return rc;
    p.tiles_n = static_cast<int32_t>((N + 255) / 256);
    cudaError_t e3 = launch_gemm_blockscaled_wide(tmA, tmB, tma_out ? &tmC : nullptr, p, st.num_sms, cs);
    if (e3 != cudaSuccess)
      return fail(TG_ERR_LAUNCH, "block-scaled GEMM (wide tile) launch failed: %s", cudaGetErrorString(e3));
    return TG_OK;
  }
  cudaError_t e = launch_gemm_blockscaled(tmA, tmB, tma_out ? &tmC : nullptr, p, st.num_sms, cs);
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "block-scaled GEMM launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

static int32_t check_dense(const TgTensorDesc* t, const char* name) {
  if (t == nullptr) return fail(TG_ERR_NULL, "%s descriptor is null", name);
  if (t->ndim < 1 || t->ndim > 5) return fail(TG_ERR_ARGS, "%s must have 1 to 5 dimensions", name);
  int64_t expect = 1;
  for (int d = t->ndim - 1; d >= 0; --d) {
    if (t->shape[d] < 0) return fail(TG_ERR_ARGS, "%s has a negative extent", name);
    if (t->shape[d] != 1 && t->strides[d] != expect) return fail(TG_ERR_ARGS, "%s must be contiguous", name);
    expect *= t->shape[d];
  }
  return TG_OK;
}
static int64_t numel(const TgTensorDesc* t) {
  int64_t n = 1;
  for (int d = 0; d < t->ndim; ++d) n *= t->shape[d];
  return n;
}
static bool is_in_dtype(int32_t d) { return d == TG_F32 || d == TG_F16 || d == TG_BF16; }

int32_t tg_act_quant(const TgTensorDesc* Y, const TgTensorDesc* S, const TgTensorDesc* X, int32_t block,
                     int32_t device_id, uint64_t stream) {
  int32_t rc;
  if ((rc = check_dense(X, "X")) != TG_OK) return rc;
  if ((rc = check_dense(Y, "Y")) != TG_OK) return rc;
  if ((rc = check_dense(S, "S")) != TG_OK) return rc;
  if (!is_in_dtype(X->dtype)) return fail(TG_ERR_DTYPE, "X must be f32, f16 or bf16");
  if (Y->dtype != TG_F8E4M3) return fail(TG_ERR_DTYPE, "Y must be float8_e4m3fn");
  if (S->dtype != TG_F32) return fail(TG_ERR_DTYPE, "S must be f32");
  if (block != 128) return fail(TG_ERR_ARGS, "only block_size 128 is implemented, got %d", block);
  const int64_t n = numel(X);
  const int64_t K = X->shape[X->ndim - 1];
  if (K % block != 0) return fail(TG_ERR_ARGS, "last dimension %lld is not a multiple of block_size %d", (long long)K, block);
  if (numel(Y) != n || numel(S) != n / block) return fail(TG_ERR_ARGS, "Y / S sizes do not match X");
  if (n == 0) return TG_OK;
  if (X->ptr == 0 || Y->ptr == 0 || S->ptr == 0) return fail(TG_ERR_NULL, "data pointer is null");
  if ((X->ptr & 15u) || (Y->ptr & 15u) || (S->ptr & 3u)) return fail(TG_ERR_ALIGN, "X and Y must be 16-byte, S 4-byte aligned");
  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  cudaError_t e = launch_act_quant(reinterpret_cast<void*>(Y->ptr), reinterpret_cast<float*>(S->ptr),
                                   reinterpret_cast<const void*>(X->ptr), X->dtype, n / block,
                                   reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "act_quant launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

int32_t tg_weight_dequant(const TgTensorDesc* Y, const TgTensorDesc* X, const TgTensorDesc* S, int32_t block,
                          int32_t device_id, uint64_t stream) {
  int32_t rc;
  if ((rc = check_dense(X, "X")) != TG_OK) return rc;
  if ((rc = check_dense(Y, "Y")) != TG_OK) return rc;
  if ((rc = check_dense(S, "S")) != TG_OK) return rc;
  if (X->dtype != TG_F8E4M3) return fail(TG_ERR_DTYPE, "X must be float8_e4m3fn");
  if (!is_out_dtype(Y->dtype)) return fail(TG_ERR_DTYPE, "Y must be f32, f16 or bf16");
  if (S->dtype != TG_F32) return fail(TG_ERR_DTYPE, "S must be f32");
  if (block != 128) return fail(TG_ERR_ARGS, "only block_size 128 is implemented, got %d", block);
  if (X->ndim != 2 || Y->ndim != 2 || S->ndim != 2) return fail(TG_ERR_ARGS, "X, Y and S must be 2-D");
  const int64_t M = X->shape[0], N = X->shape[1];
  if (Y->shape[0] != M || Y->shape[1] != N) return fail(TG_ERR_ARGS, "Y must have X's shape");
  if (S->shape[0] != (M + 127) / 128 || S->shape[1] != (N + 127) / 128)
    return fail(TG_ERR_ARGS, "S must be [ceil(M/128), ceil(N/128)]");
  if (M == 0 || N == 0) return TG_OK;
  if (X->ptr == 0 || Y->ptr == 0 || S->ptr == 0) return fail(TG_ERR_NULL, "data pointer is null");
  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  cudaError_t e = launch_weight_dequant(reinterpret_cast<void*>(Y->ptr), Y->dtype, reinterpret_cast<const uint8_t*>(X->ptr),
                                        reinterpret_cast<const float*>(S->ptr), M, N, S->shape[1],
                                        reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "weight_dequant launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

int32_t tg_quant_pertensor(const TgTensorDesc* Y, uint64_t scale_out, const TgTensorDesc* X, uint64_t amax_scratch,
                           int32_t device_id, uint64_t stream) {
  int32_t rc;
  if ((rc = check_dense(X, "X")) != TG_OK) return rc;
  if ((rc = check_dense(Y, "Y")) != TG_OK) return rc;
  if (!is_in_dtype(X->dtype)) return fail(TG_ERR_DTYPE, "X must be f32, f16 or bf16");
  if (Y->dtype != TG_F8E4M3) return fail(TG_ERR_DTYPE, "Y must be float8_e4m3fn");
  if (scale_out == 0 || amax_scratch == 0) return fail(TG_ERR_NULL, "scale_out / amax_scratch pointer is null");
  if ((scale_out & 3u) || (amax_scratch & 3u)) return fail(TG_ERR_ALIGN, "scale_out / amax_scratch must be 4-byte aligned");
  const int64_t n = numel(X);
  if (numel(Y) != n) return fail(TG_ERR_ARGS, "Y must have as many elements as X");
  if (n > 0 && (X->ptr == 0 || Y->ptr == 0)) return fail(TG_ERR_NULL, "data pointer is null");
  if ((X->ptr & 15u) || (Y->ptr & 3u)) return fail(TG_ERR_ALIGN, "X must be 16-byte and Y 4-byte aligned");
  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  cudaError_t e = launch_quant_pertensor(reinterpret_cast<uint8_t*>(Y->ptr), reinterpret_cast<float*>(scale_out),
                                         reinterpret_cast<const void*>(X->ptr), X->dtype, n,
                                         reinterpret_cast<uint32_t*>(amax_scratch), g_dev[device_id].num_sms,
                                         knob(kKnobQuantFused, 1) != 0,  // TILEGYM_B200_QUANT_FUSED=0: always two passes
                                         reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "quant_pertensor launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

int32_t tg_weight_quant_block(const TgTensorDesc* Y, const TgTensorDesc* S, const TgTensorDesc* X, int32_t block,
                              int32_t device_id, uint64_t stream) {
  int32_t rc;
  if ((rc = check_dense(X, "X")) != TG_OK) return rc;
  if ((rc = check_dense(Y, "Y")) != TG_OK) return rc;
  if ((rc = check_dense(S, "S")) != TG_OK) return rc;
  if (!is_in_dtype(X->dtype)) return fail(TG_ERR_DTYPE, "X must be f32, f16 or bf16");
  if (Y->dtype != TG_F8E4M3) return fail(TG_ERR_DTYPE, "Y must be float8_e4m3fn");
  if (S->dtype != TG_F32) return fail(TG_ERR_DTYPE, "S must be f32");
  if (block != 128) return fail(TG_ERR_ARGS, "only block_size 128 is implemented, got %d", block);
  if (X->ndim != 2 || Y->ndim != 2 || S->ndim != 2) return fail(TG_ERR_ARGS, "X, Y and S must be 2-D");
  const int64_t N = X->shape[0], K = X->shape[1];
  if (Y->shape[0] != N || Y->shape[1] != K) return fail(TG_ERR_ARGS, "Y must have X's shape");
  if (S->shape[0] != (N + 127) / 128 || S->shape[1] != (K + 127) / 128)
    return fail(TG_ERR_ARGS, "S must be [ceil(N/128), ceil(K/128)]");
  if (N == 0 || K == 0) return TG_OK;
  if (X->ptr == 0 || Y->ptr == 0 || S->ptr == 0) return fail(TG_ERR_NULL, "data pointer is null");
  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  cudaError_t e = launch_weight_quant_block(reinterpret_cast<uint8_t*>(Y->ptr), reinterpret_cast<float*>(S->ptr),
                                            reinterpret_cast<const void*>(X->ptr), X->dtype, N, K, S->shape[1],
                                            reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "weight_quant_block launch failed: %s", cudaGetErrorString(e));
  return TG_OK;
}

int32_t tg_device_status(int32_t device_id, int32_t* detail) {
  if (detail) *detail = 0;
  DeviceGuard guard(device_id);
  if (guard.err != cudaSuccess) {
    cudaGetLastError();
    return fail(TG_ERR_DEVICE, "cannot select CUDA device %d", device_id);
  }
  int32_t rc;
  if ((rc = init_device(device_id)) != TG_OK) return rc;
  int32_t word = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&word, g_dev[device_id].status, sizeof(word), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(TG_ERR_LAUNCH, "device %d reports: %s", device_id, cudaGetErrorString(e));
  if (word != 0) {
    int32_t zero = 0;
    cudaMemcpy(g_dev[device_id].status, &zero, sizeof(zero), cudaMemcpyHostToDevice);
    if (detail) *detail = word;
    return fail(TG_ERR_TIMEOUT, "a bounded device-side wait expired (role %d, site %d)", word / 1000, word % 1000);
  }
  return TG_OK;
}

}  // extern "C"

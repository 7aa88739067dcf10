// Host-side utilities of libb200attn: thread-local error text, TMA tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda), dropout threshold.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace b200attn {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return B200ATTN_ECUDA;
}

const char* last_error() { return g_err; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

int check_tma_operand(const b200attn_tensor& t, int elem_bytes, const char* name) {
  if (t.ptr == nullptr) {
    set_error("%s: null pointer", name);
    return B200ATTN_EINVAL;
  }
  if (reinterpret_cast<uintptr_t>(t.ptr) % 16 != 0) {
    set_error("%s: base address must be 16-byte aligned", name);
    return B200ATTN_EINVAL;
  }
  if (t.stride[3] != 1) {
    set_error("%s: feature stride must be 1 (got %lld)", name, static_cast<long long>(t.stride[3]));
    return B200ATTN_EINVAL;
  }
  return B200ATTN_OK;
}

int encode_tmap_4d(CUtensorMap* out, const b200attn_tensor& t, int elem_bytes, int64_t B, int64_t H,
                   int64_t rows, int64_t D, int box_cols, int box_rows, int swizzle,
                   const char* name, int box_heads) {
  int rc = check_tma_operand(t, elem_bytes, name);
  if (rc != B200ATTN_OK) return rc;
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return B200ATTN_ECUDA;
  }
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  const int64_t ext[3] = {rows, H, B};
  const int64_t raw[3] = {t.stride[2], t.stride[1], t.stride[0]};
  cuuint64_t strides[3];
  int64_t fallback = D * elem_bytes;
  for (int i = 0; i < 3; ++i) {
    int64_t sb = raw[i] * elem_bytes;
    if (ext[i] == 1) {
      // The stride of an extent-1 dimension is never used for addressing; any legal value works.
      if (sb <= 0 || sb % 16 != 0) sb = fallback;
    }
    if (sb <= 0 || sb % 16 != 0 || sb >= (1ll << 40)) {
      set_error("%s: stride %lld bytes of dim %d is not a positive multiple of 16 below 2^40", name,
                static_cast<long long>(sb), 2 - i);
      return B200ATTN_EINVAL;
    }
    strides[i] = static_cast<cuuint64_t>(sb);
    fallback = sb * (ext[i] > 0 ? ext[i] : 1);
    if (fallback % 16 != 0 || fallback >= (1ll << 40)) fallback = D * elem_bytes;
  }
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows),
                             static_cast<cuuint32_t>(box_heads), 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUtensorMapDataType dt =
      elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  CUresult r = fn(out, dt, 4, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  static_cast<CUtensorMapSwizzle>(swizzle), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("%s: cuTensorMapEncodeTiled failed with CUresult %d (dims %lld,%lld,%lld,%lld box %d,%d)",
              name, static_cast<int>(r), static_cast<long long>(D), static_cast<long long>(rows),
              static_cast<long long>(H), static_cast<long long>(B), box_cols, box_rows);
    return B200ATTN_ECUDA;
  }
  return B200ATTN_OK;
}

int32_t dropout_keep_threshold(float dropout_p) {
  // Largest x in [0, 2^31) with float(x) * scale <= p, or -1 when every x is kept.
  const float scale = 4.6566127342e-10f;
  auto dropped = [&](int64_t x) {
    volatile float u = static_cast<float>(static_cast<int32_t>(x)) * scale;
    return !(u > dropout_p);
  };
  if (!dropped(0)) return -1;
  int64_t lo = 0, hi = (1ll << 31) - 1;  // dropped(lo) is true
  if (dropped(hi)) return static_cast<int32_t>(hi);
  while (hi - lo > 1) {
    const int64_t mid = lo + (hi - lo) / 2;
    if (dropped(mid)) lo = mid; else hi = mid;
  }
  return static_cast<int32_t>(lo);
}

}  // namespace b200attn

extern "C" {
int b200attn_abi_version(void) { return B200ATTN_ABI_VERSION; }
const char* b200attn_last_error(void) { return b200attn::last_error(); }
}

// Host-side check of the prepared divisions behind the kernels' work-item order: every id of a grid
// of `pairs` (batch, head) pairs x `n_z` row blocks in chunks of `chunk` pairs must decode to the
// pair and block that plain integer division gives. Returns the number of ids that do not.
extern "C" int b200attn_work_order_selftest(int32_t pairs, int32_t n_z, int32_t chunk) {
  using namespace b200attn;
  if (pairs <= 0 || n_z <= 0 || chunk <= 0 || static_cast<int64_t>(pairs) * n_z > 0x7fffffff) {
    set_error("work_order_selftest: bad argument");
    return B200ATTN_EINVAL;
  }
  const BlockOrder order = BlockOrder::make(pairs, n_z, chunk);
  const int per_chunk = chunk * n_z, full = pairs / chunk;
  int bad = 0;
  for (int id = 0; id < pairs * n_z; ++id) {
    int c = id / per_chunk, width = chunk;
    if (c >= full) { c = full; width = pairs - full * chunk; }
    const int rem = id - c * per_chunk;
    const int z = rem / width, bh = c * chunk + rem - z * width;
    const BlockCoord got = order.decode(id);
    if (got.z != z || got.bh != bh) ++bad;
  }
  const FastDiv by_pairs = FastDiv::make(pairs);
  for (int64_t n = 0; n < 0x7fffffff; n += 1 + n / 97) {
    if (by_pairs.div(static_cast<int>(n)) != static_cast<int>(n / pairs)) ++bad;
  }
  if (by_pairs.div(0x7fffffff) != 0x7fffffff / pairs) ++bad;
  return bad;
}

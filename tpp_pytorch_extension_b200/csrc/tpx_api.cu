// C-ABI entry points that are not tied to one kernel file: error text, device info, and the
// dispatch of tpx_qlinear onto the kernel families.
#include "tpx_common.cuh"
#include <string.h>
#include <stdlib.h>

namespace tpx {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static unsigned long long g_launches = 0;  // relaxed tally; exact when one host thread launches
void count_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }

static Knobs g_knobs;
static bool g_knobs_read = false;

static void read_knobs() {
  auto env = [](const char* name, int dflt) { const char* e = getenv(name); return e ? atoi(e) : dflt; };
  g_knobs.tc_whole = env("TPX_TC_WHOLE", -1);
  g_knobs.tc_wide = env("TPX_TC_WIDE", -1);
  g_knobs.tc_f4 = env("TPX_TC_F4", -1);
  g_knobs.tc_w4 = env("TPX_TC_W4", -1);
  g_knobs.tc4_occ = env("TPX_TC4_OCC", 1);
  g_knobs.tc_cluster = env("TPX_TC_CLUSTER", 1);
  g_knobs.tc_pf = env("TPX_TC_PF", 0);
  g_knobs.handoff_min = env("TPX_HANDOFF_MIN_TOKENS", 33);
  g_knobs.tc_p = env("TPX_TC_P", -1);
  g_knobs.tc_p2 = env("TPX_TC_P2", -1);
  g_knobs.tc_p_rows = env("TPX_TC_P_ROWS", 1);
  g_knobs.tc_p_uks = env("TPX_TC_P_UKS", 2);
  g_knobs.attn_splits = env("TPX_ATTN_SPLITS", 0);
  g_knobs.attn_tc = env("TPX_ATTN_TC", 1);
#ifdef TPX_DEBUG
  g_knobs.dbg = env("TPX_TC_DBG", 0);
#else
  g_knobs.dbg = 0;
#endif
  g_knobs_read = true;
}

const Knobs& knobs() {
  if (!g_knobs_read) read_knobs();
  return g_knobs;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

size_t qlinear_stream_scratch_bytes(int kind, int64_t M, int64_t N, int64_t K, int64_t block_size, bool dual);
int qlinear_stream_launch(int kind, const uint8_t* pk_codes, const void* pk_scales, const uint8_t* pk_codes2,
                          const void* pk_scales2, int64_t block_size, const uint16_t* x, int64_t M, int64_t N, int64_t K,
                          const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res, float res_scale,
                          uint16_t* y, void* scratch, size_t scratch_bytes, cudaStream_t st);

__global__ void e2m1_pair_table_kernel(uint32_t* out) {
  uint32_t b = threadIdx.x;
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(b));
  out[b] = r;
}

}  // namespace tpx

using namespace tpx;

extern "C" int tpx_version(void) { return 100; }
extern "C" const char* tpx_last_error(void) { return g_err; }
extern "C" int tpx_sm_count(void) { return sm_count(); }
extern "C" void tpx_reload_options(void) { read_knobs(); }

extern "C" int tpx_e2m1_pair_table(uint32_t* out256, void* stream) {
  TPX_REQUIRE(out256, TPX_ERR_ARG, "e2m1_pair_table: null pointer");
  e2m1_pair_table_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(out256);
  TPX_LAUNCH_OK();
  return TPX_OK;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_qlinear_shape(int kind, int64_t M, int64_t N, int64_t K, int64_t block_size) {
  TPX_REQUIRE(kind == TPX_W_MXFP4 || kind == TPX_W_INT8, TPX_ERR_ARG, "qlinear: unknown weight kind %d", kind);
  TPX_REQUIRE(M >= 0 && N > 0 && K > 0, TPX_ERR_ARG, "qlinear: bad shape M=%ld N=%ld K=%ld", (long)M, (long)N, (long)K);
  TPX_REQUIRE(N % 16 == 0 && K % 64 == 0, TPX_ERR_ARG, "qlinear: needs N %% 16 == 0 and K %% 64 == 0 (N=%ld K=%ld)", (long)N, (long)K);
  TPX_REQUIRE(M <= INT32_MAX / 2 && N <= INT32_MAX / 2 && K <= INT32_MAX / 2 && M * N < ((int64_t)1 << 40), TPX_ERR_ARG, "qlinear: shape too large");
  if (kind == TPX_W_INT8)
    TPX_REQUIRE(block_size >= 64 && block_size % 64 == 0 && K % block_size == 0, TPX_ERR_ARG,
                "qlinear: int8 block size %ld must be a multiple of 64 dividing K=%ld", (long)block_size, (long)K);
  return TPX_OK;
}

extern "C" size_t tpx_qlinear_scratch_bytes(int kind, int64_t M, int64_t N, int64_t K, int64_t block_size, int dual) {
  if (check_qlinear_shape(kind, M, N, K, block_size) != TPX_OK) return 0;
  if (M == 0) return 0;
  return qlinear_stream_scratch_bytes(kind, M, N, K, block_size, dual != 0);
}

extern "C" int tpx_qlinear(int kind, const uint8_t* pk_codes, const void* pk_scales, const uint8_t* pk_codes2,
                           const void* pk_scales2, int64_t block_size, const uint16_t* x, int64_t M, int64_t N,
                           int64_t K, const uint16_t* bias, int act, const uint16_t* mul_in, const uint16_t* res,
                           float res_scale, uint16_t* y, void* scratch, size_t scratch_bytes, void* stream) {
  int rc = check_qlinear_shape(kind, M, N, K, block_size);
  if (rc != TPX_OK) return rc;
  if (M == 0) return TPX_OK;  // empty batch: nothing to do, as a zero-row GEMM in the reference
  TPX_REQUIRE(pk_codes && x && y, TPX_ERR_ARG, "qlinear: null pointer");
  if (kind == TPX_W_INT8) {  // MXFP4 tiles carry their scales; int8 scales are a separate array
    TPX_REQUIRE(pk_scales, TPX_ERR_ARG, "qlinear: int8 needs the scale array");
    TPX_REQUIRE((pk_codes2 == nullptr) == (pk_scales2 == nullptr), TPX_ERR_ARG, "qlinear: second weight needs both codes and scales");
  }
  TPX_REQUIRE(!(pk_codes2 && mul_in), TPX_ERR_ARG, "qlinear: gate/up pair and mul_in are exclusive");
  TPX_REQUIRE(act >= TPX_ACT_NONE && act <= TPX_ACT_RELU, TPX_ERR_ARG, "qlinear: unknown activation %d", act);
  TPX_REQUIRE(aligned16(pk_codes) && aligned16(pk_scales) && aligned16(x) && aligned16(pk_codes2) && aligned16(pk_scales2),
              TPX_ERR_ARG, "qlinear: weights and activations must be 16-byte aligned");
  return qlinear_stream_launch(kind, pk_codes, pk_scales, pk_codes2, pk_scales2, block_size, x, M, N, K, bias, act, mul_in,
                        res, res_scale, y, scratch, scratch_bytes, (cudaStream_t)stream);
}

extern "C" unsigned long long tpx_launch_count(void) { return __atomic_load_n(&tpx::g_launches, __ATOMIC_RELAXED); }

#include "common.cuh"

#include <atomic>

namespace paro {

static std::atomic<long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

char* error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int check_tensor(const char* name, const void* p, int dtype, int B, int H, int N, int D,
                 int64_t sb, int64_t sh, int64_t sn) {
  PARO_REQUIRE(p != nullptr, PARO_EINVAL, "%s: null pointer", name);
  PARO_REQUIRE(dtype == PARO_F16 || dtype == PARO_BF16, PARO_EINVAL, "%s: dtype must be fp16 or bf16", name);
  PARO_REQUIRE(B > 0 && H > 0 && N > 0, PARO_ESHAPE, "%s: empty tensor (B=%d H=%d N=%d)", name, B, H, N);
  PARO_REQUIRE(D == 64 || D == 128, PARO_ESHAPE, "%s: head_dim %d unsupported (64 or 128)", name, D);
  PARO_REQUIRE(aligned16(p), PARO_EALIGN, "%s: pointer not 16-byte aligned", name);
  PARO_REQUIRE(sb % 8 == 0 && sh % 8 == 0 && sn % 8 == 0, PARO_EALIGN,
               "%s: strides must be multiples of 8 elements", name);
  PARO_REQUIRE(sn >= D, PARO_ESHAPE, "%s: token stride %lld smaller than head_dim", name, (long long)sn);
  return PARO_OK;
}

}  // namespace paro

extern "C" int paro_version(void) { return 100; }
extern "C" long long paro_launch_count(void) { return paro::launches(); }
extern "C" const char* paro_last_error(void) { return paro::error_buffer(); }

// Status strings, device checks and the CPU-only self test of the unpack tables.
#include <cstdio>
#include <cstring>
#include <random>

#include "nb_common.cuh"
#include "nb_host.h"

namespace nb {

static thread_local char g_last_error[256] = "";

int record_cuda_error(cudaError_t e) {
  if (e == cudaSuccess) return NB_OK;
  std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return NB_ERR_LAUNCH;
}

void set_last_error(const char* msg) { std::snprintf(g_last_error, sizeof(g_last_error), "%s", msg); }

static int g_cc_major[64];
static int g_sms[64];
static bool g_known[64];

static int query_device(int* dev_out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (dev < 0 || dev >= 64) return NB_ERR_ARG;
  if (!g_known[dev]) {
    int major = 0, sms = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    g_cc_major[dev] = major;
    g_sms[dev] = sms;
    g_known[dev] = true;
  }
  *dev_out = dev;
  return NB_OK;
}

int check_device() {
  int dev;
  if (int rc = query_device(&dev)) return rc;
  return g_cc_major[dev] == 10 ? NB_OK : NB_ERR_ARCH;
}

int sm_count() {
  int dev;
  if (query_device(&dev)) return 148;
  return g_sms[dev] > 0 ? g_sms[dev] : 148;
}

int check_launch() { return record_cuda_error(cudaGetLastError()); }

// Packs `idx` (128 indices) the way the reference does and checks that the selector words
// give the index back at every slot.
template <int BITS> static bool selftest_bits(std::mt19937& rng) {
  for (int trial = 0; trial < 200; ++trial) {
    uint8_t idx[kBlock];
    for (int i = 0; i < kBlock; ++i) idx[i] = (uint8_t)(rng() & ((1u << BITS) - 1u));
    if (trial == 0) for (int i = 0; i < kBlock; ++i) idx[i] = (uint8_t)(i & ((1u << BITS) - 1u));
    uint32_t w[Fmt<BITS>::kWords];
    std::memset(w, 0, sizeof(w));
    for (int i = 0; i < kBlock; ++i) {  // LSB-first bit stream
      const int bit = i * BITS;
      w[bit >> 5] |= (uint32_t)idx[i] << (bit & 31);
      if ((bit & 31) + BITS > 32) w[(bit >> 5) + 1] |= (uint32_t)idx[i] >> (32 - (bit & 31));
    }
    bool seen[kBlock] = {false};
    for (int q = 0; q < 4; ++q) {
      uint32_t U[4];
      group_selectors<BITS>(w, q, U);
      for (int u = 0; u < 4; ++u) {
        if (BITS < 4 && (U[u] & 0x88888888u)) return false;  // bit 3 of every nibble must be clear (it belongs to the index at 4 bits)
        for (int k = 0; k < 8; ++k) {
          const int pos = slot_position<BITS>(q, u, k);
          if (pos < 0 || pos >= kBlock || seen[pos]) return false;
          seen[pos] = true;
          if (((U[u] >> (4 * k)) & 0xFu) != idx[pos]) return false;
          const int slot = 4 * (8 * q + 2 * u + (k >> 2)) + (k & 3);
          if (slot_to_position<BITS>(slot) != pos) return false;
        }
      }
    }
  }
  return true;
}

}  // namespace nb

extern "C" int nb_version(void) { return 100; }

extern "C" const char* nb_status_string(int s) {
  switch (s) {
    case NB_OK: return "ok";
    case NB_ERR_ARG: return "invalid argument";
    case NB_ERR_ALIGN: return "pointer not 16-byte aligned";
    case NB_ERR_SHAPE: return "shape not supported";
    case NB_ERR_ARCH: return "device is not sm_100";
    case NB_ERR_LAUNCH: return "CUDA launch failed";
    case NB_ERR_TIMEOUT: return "device-side wait timed out";
    case NB_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

extern "C" const char* nb_last_cuda_error(void) { return nb::g_last_error; }

extern "C" int nb_selftest_tables(void) {
  std::mt19937 rng(1234);
  if (!nb::selftest_bits<3>(rng)) return NB_ERR_SHAPE;
  if (!nb::selftest_bits<2>(rng)) return NB_ERR_SHAPE;
  if (!nb::selftest_bits<4>(rng)) return NB_ERR_SHAPE;
  return NB_OK;
}

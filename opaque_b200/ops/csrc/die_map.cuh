// Which SMs share a die with which?  (B200: 148 SMs on two dies, each die with its own half of the L2.)
//
// A line of global memory has one home L2 slice.  Atomics execute at the home slice, so their round trip from an SM
// is short when the slice sits on the SM's own die (about 280 clocks measured) and long when the request crosses the
// die-to-die link (650 - 750 clocks).  Every SM times an atomic on each of DM_LINES scattered lines (minimum of a few
// repetitions); two SMs on the same die see the same near / far pattern over the lines (correlation +1), two SMs on
// different dies the opposite one (correlation -1).  SM ids do not map to dies in a regular way and the map differs
// from GPU to GPU (floor sweeping), hence a measurement, once per device and process (under a millisecond).
//
// The probe has no waits and touches only its own static buffers; it allocates nothing.  Used by the CTA-pair GEMM to
// keep the tiles that share operands on one die.  No counterpart in the reference (its GEMMs are library calls).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cmath>
#include <mutex>
#include <vector>

namespace ob {

constexpr int DM_LINES = 192;
constexpr int DM_STRIDE_WORDS = (4096 + 128) / 4;      // distance between probed lines: different slices and sets
constexpr int DM_REPS = 6;
constexpr int DM_MAX_SMS = 256;

static __device__ unsigned int g_dm_lines[DM_LINES * DM_STRIDE_WORDS];
static __device__ unsigned int g_dm_lat[DM_MAX_SMS * DM_LINES];
static __device__ int g_dm_smid[DM_MAX_SMS];
static __device__ unsigned char g_sm_die[DM_MAX_SMS];   // smid -> 0 / 1, all zero until (or without) a successful probe

// One CTA per SM (the launch asks for enough shared memory that two cannot share one); thread 0 measures.
__global__ void __launch_bounds__(32, 1) die_probe_kernel() {
  if (threadIdx.x != 0 || blockIdx.x >= DM_MAX_SMS) return;
  unsigned smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  g_dm_smid[blockIdx.x] = static_cast<int>(smid);
  unsigned sink = 0;
  for (int i = 0; i < DM_LINES; ++i) {
    const int line = (i + 13 * blockIdx.x) % DM_LINES;   // SMs walk the lines at different offsets: less queueing
    unsigned int* a = g_dm_lines + static_cast<size_t>(line) * DM_STRIDE_WORDS;
    unsigned best = 0xffffffffu;
    for (int r = 0; r < DM_REPS; ++r) {
      unsigned long long dd;
      unsigned old;
      // The atomic's address depends on the first clock read and the second clock read is predicated on the value the
      // atomic returns, so neither read can move across it.
      asm volatile(
          "{\n\t"
          ".reg .u64 t0, t1, addr, off;\n\t"
          ".reg .u32 old;\n\t"
          ".reg .pred p;\n\t"
          "mov.u64 t0, %%clock64;\n\t"
          "shr.u64 off, t0, 63;\n\t"
          "shl.b64 off, off, 2;\n\t"
          "add.u64 addr, %2, off;\n\t"
          "atom.global.add.u32 old, [addr], 1;\n\t"
          "setp.ne.u32 p, old, 0xffffffff;\n\t"
          "mov.u64 t1, t0;\n\t"
          "@p mov.u64 t1, %%clock64;\n\t"
          "sub.u64 %0, t1, t0;\n\t"
          "mov.u32 %1, old;\n\t"
          "}"
          : "=l"(dd), "=r"(old)
          : "l"(a)
          : "memory");
      sink += old;
      const unsigned d = static_cast<unsigned>(dd);
      best = d < best ? d : best;
    }
    g_dm_lat[blockIdx.x * DM_LINES + line] = best;
  }
  if (sink == 0x12345678u) g_dm_lines[0] = sink;
}

struct DieMap {
  bool probed = false;     // a probe ran (successfully or not); it is not repeated
  bool valid = false;      // two groups were found and the table on the device is filled
  int sms = 0;
  int tpcs[2] = {0, 0};    // SM pairs per die
  std::vector<unsigned char> die;   // by smid
};

// Classifies on the host.  Returns false (map stays all-zero: every SM "die 0", i.e. no die-aware scheduling) when the
// latencies do not split cleanly into two groups.
static bool dm_classify(const std::vector<int>& smid, const std::vector<unsigned>& lat, int blocks, DieMap* out) {
  int ref = 0;
  for (int b = 0; b < blocks; ++b)
    if (smid[b] < smid[ref]) ref = b;
  auto corr = [&](int a, int b) {
    double ma = 0, mb = 0;
    for (int i = 0; i < DM_LINES; ++i) {
      ma += lat[a * DM_LINES + i];
      mb += lat[b * DM_LINES + i];
    }
    ma /= DM_LINES;
    mb /= DM_LINES;
    double sab = 0, saa = 0, sbb = 0;
    for (int i = 0; i < DM_LINES; ++i) {
      const double x = lat[a * DM_LINES + i] - ma, y = lat[b * DM_LINES + i] - mb;
      sab += x * y;
      saa += x * x;
      sbb += y * y;
    }
    return sab / std::sqrt(saa * sbb + 1e-9);
  };
  out->die.assign(DM_MAX_SMS, 0);
  int count[2] = {0, 0};
  for (int b = 0; b < blocks; ++b) {
    const double c = corr(ref, b);
    if (c > -0.6 && c < 0.6) return false;             // not bimodal: a single-die part, or a disturbed measurement
    if (smid[b] < 0 || smid[b] >= DM_MAX_SMS) return false;
    const int d = c < 0 ? 1 : 0;
    out->die[smid[b]] = static_cast<unsigned char>(d);
    ++count[d];
  }
  if (count[0] == 0 || count[1] == 0) return false;
  // the two SMs of a pair (2t, 2t + 1) must agree: the pair kernels place one cluster on such a pair
  for (int s = 0; s + 1 < DM_MAX_SMS; s += 2)
    if (out->die[s] != out->die[s + 1]) {
      bool both_seen = false;
      for (int b = 0; b < blocks; ++b)
        if (smid[b] == s + 1) both_seen = true;
      if (both_seen) return false;
    }
  out->tpcs[0] = count[0] / 2;
  out->tpcs[1] = count[1] / 2;
  return true;
}

// The map of the current device; probes on first use.  Must not run while a stream capture is active on this thread
// (the caller checks); the probe synchronises the device.
static const DieMap& die_map_for_current_device() {
  static DieMap maps[64];
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::lock_guard<std::mutex> lock(mu);
  DieMap& m = maps[dev];
  if (m.probed) return m;
  m.probed = true;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0 || sms > DM_MAX_SMS) return m;
  m.sms = sms;
  constexpr int probe_smem = 160 * 1024;               // more than half an SM's shared memory: one CTA per SM
  if (cudaFuncSetAttribute(die_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, probe_smem) != cudaSuccess) {
    cudaGetLastError();
    return m;
  }
  for (int pass = 0; pass < 2; ++pass) die_probe_kernel<<<sms, 32, probe_smem>>>();      // first pass warms the lines
  std::vector<int> smid(sms);
  std::vector<unsigned> lat(static_cast<size_t>(sms) * DM_LINES);
  if (cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemcpyFromSymbol(smid.data(), g_dm_smid, sms * sizeof(int)) != cudaSuccess ||
      cudaMemcpyFromSymbol(lat.data(), g_dm_lat, lat.size() * sizeof(unsigned)) != cudaSuccess) {
    cudaGetLastError();
    return m;
  }
  if (!dm_classify(smid, lat, sms, &m)) {
    m.die.assign(DM_MAX_SMS, 0);
    return m;
  }
  if (cudaMemcpyToSymbol(g_sm_die, m.die.data(), DM_MAX_SMS) != cudaSuccess) {
    cudaGetLastError();
    m.die.assign(DM_MAX_SMS, 0);
    return m;
  }
  m.valid = true;
  return m;
}

}  // namespace ob

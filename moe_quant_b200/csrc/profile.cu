#include "profile.cuh"
#include "../../include/moequant_bench.h"

#include <vector>

namespace mq {

bool g_profile_on = false;

namespace {
struct Sample {
  cudaEvent_t a, b;
  int kind;
  double work, work2;
};
std::vector<Sample> g_samples;
std::vector<cudaEvent_t> g_pool;
constexpr size_t kMaxSamples = 1 << 16;

cudaEvent_t take_event() {
  if (!g_pool.empty()) {
    cudaEvent_t e = g_pool.back();
    g_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
}  // namespace

void prof_open(int kind, double work, double work2, cudaStream_t st) {
  if (g_samples.size() >= kMaxSamples) return;
  Sample s;
  s.a = take_event();
  s.b = nullptr;
  s.kind = kind;
  s.work = work;
  s.work2 = work2;
  cudaEventRecord(s.a, st);
  g_samples.push_back(s);
}

void prof_close(cudaStream_t st) {
  if (g_samples.empty() || g_samples.back().b != nullptr) return;
  g_samples.back().b = take_event();
  cudaEventRecord(g_samples.back().b, st);
}

}  // namespace mq

extern "C" long long mq_launch_count(void) { return mq::g_launches; }

extern "C" int mq_profile_begin(void) {
  mq::g_profile_on = true;
  return MQ_OK;
}

// Synchronises the device, then sums per kind.  Each array has MQ_PROFILE_KINDS entries.
extern "C" int mq_profile_end(int64_t* launches, double* milliseconds, double* work, double* work2) {
  using namespace mq;
  g_profile_on = false;
  MQ_REQUIRE(launches && milliseconds && work && work2, MQ_ERR_ARGUMENT, "mq_profile_end: null pointer");
  MQ_CUDA(cudaDeviceSynchronize());
  for (int k = 0; k < PROF_KINDS; ++k) {
    launches[k] = 0;
    milliseconds[k] = work[k] = work2[k] = 0.0;
  }
  for (Sample& s : g_samples) {
    if (s.b) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, s.a, s.b) == cudaSuccess) {
        launches[s.kind] += 1;
        milliseconds[s.kind] += ms;
        work[s.kind] += s.work;
        work2[s.kind] += s.work2;
      }
      g_pool.push_back(s.b);
    }
    g_pool.push_back(s.a);
  }
  g_samples.clear();
  return MQ_OK;
}

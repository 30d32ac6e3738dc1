// Host-side runtime pieces that must not depend on the Python interpreter.
//
// 1. Status watchdog. Every kernel of this library that waits on another agent (a TMA, an MMA, a
//    peer GPU) bounds its wait and, when the limit runs out, writes an error code into a per-device
//    status word and leaves in an orderly way. Reading that word from Python costs a device
//    synchronisation, so training loops look at it rarely. The watchdog is a C++ thread (no GIL)
//    that copies the word to pinned host memory on its own stream every `interval_ms` and keeps the
//    first non-zero code together with the time it was seen; Python asks for it without touching
//    the device (`nb_rt_watch_last`). It never resets, faults or blocks the device: it only reads.
//
// 2. Step pacing statistics: the same thread timestamps every poll, so the host can tell how long
//    the device has been unresponsive to a 4-byte copy (a stuck collective shows up as a poll that
//    does not return; `nb_rt_watch_stalled_ms` reports the age of the oldest outstanding poll).
//
// The reference framework has no counterpart (its runtime is the closed MAX engine); this is the
// one-process-per-GPU replacement for "the executor notices that a device stopped answering".
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>

namespace {

struct Watch {
  std::thread th;
  std::atomic<bool> stop{false};
  std::atomic<int> code{0};            // first non-zero status seen
  std::atomic<long long> seen_ns{0};   // steady-clock time of that observation
  std::atomic<long long> polls{0};
  std::atomic<long long> poll_started_ns{0};   // 0 when no poll is outstanding
  int device = 0;
  const int* dev_word = nullptr;
  int interval_ms = 50;
};

std::mutex g_mu;
Watch* g_watch[64] = {nullptr};

long long now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

void run(Watch* w) {
  if (cudaSetDevice(w->device) != cudaSuccess) return;
  cudaStream_t s = nullptr;
  int* pinned = nullptr;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) return;
  if (cudaHostAlloc(reinterpret_cast<void**>(&pinned), sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
    cudaStreamDestroy(s);
    return;
  }
  while (!w->stop.load(std::memory_order_relaxed)) {
    w->poll_started_ns.store(now_ns(), std::memory_order_relaxed);
    *pinned = 0;
    if (cudaMemcpyAsync(pinned, w->dev_word, sizeof(int), cudaMemcpyDeviceToHost, s) == cudaSuccess &&
        cudaStreamSynchronize(s) == cudaSuccess) {
      w->polls.fetch_add(1, std::memory_order_relaxed);
      if (*pinned != 0 && w->code.load(std::memory_order_relaxed) == 0) {
        w->seen_ns.store(now_ns(), std::memory_order_relaxed);
        w->code.store(*pinned, std::memory_order_release);
      }
    } else {
      cudaGetLastError();
    }
    w->poll_started_ns.store(0, std::memory_order_relaxed);
    std::this_thread::sleep_for(std::chrono::milliseconds(w->interval_ms));
  }
  cudaFreeHost(pinned);
  cudaStreamDestroy(s);
}

}  // namespace

extern "C" {

// Start (or restart) the watchdog of `device` on the 4-byte status word at `dev_word`.
int nb_rt_watch_start(int device, const void* dev_word, int interval_ms) {
  if (device < 0 || device >= 64 || dev_word == nullptr) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_watch[device] != nullptr) {
    g_watch[device]->stop.store(true);
    if (g_watch[device]->th.joinable()) g_watch[device]->th.join();
    delete g_watch[device];
  }
  Watch* w = new Watch();
  w->device = device;
  w->dev_word = static_cast<const int*>(dev_word);
  w->interval_ms = interval_ms > 0 ? interval_ms : 50;
  w->th = std::thread(run, w);
  g_watch[device] = w;
  return 0;
}

int nb_rt_watch_stop(int device) {
  if (device < 0 || device >= 64) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  Watch* w = g_watch[device];
  if (w == nullptr) return 0;
  w->stop.store(true);
  if (w->th.joinable()) w->th.join();
  delete w;
  g_watch[device] = nullptr;
  return 0;
}

// First non-zero status code the watchdog has seen on `device` (0: none, -1: no watchdog).
int nb_rt_watch_last(int device) {
  if (device < 0 || device >= 64) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  return g_watch[device] ? g_watch[device]->code.load(std::memory_order_acquire) : -1;
}

long long nb_rt_watch_polls(int device) {
  if (device < 0 || device >= 64) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  return g_watch[device] ? g_watch[device]->polls.load() : -1;
}

// Age in milliseconds of the poll that is outstanding right now (0: none outstanding).
double nb_rt_watch_stalled_ms(int device) {
  if (device < 0 || device >= 64) return -1.0;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_watch[device]) return -1.0;
  const long long t = g_watch[device]->poll_started_ns.load();
  return t == 0 ? 0.0 : (now_ns() - t) / 1e6;
}

// Forget the recorded code (after the caller has handled it and cleared the device word).
int nb_rt_watch_clear(int device) {
  if (device < 0 || device >= 64) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_watch[device]) g_watch[device]->code.store(0);
  return 0;
}

}  // extern "C"

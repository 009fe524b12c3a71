// Host model of the device-side flag protocols, meant to run under ThreadSanitizer.
//
// The peer-memory kernels order their accesses with int32 flags: a release store into a peer's signal pad, an
// acquire poll by the owner (READY / CONSUMED / VERSION of the ZeRO-3 path, csrc/comm_kernels.cu; DISPATCH / COMBINE
// epochs of the expert-parallel layer, csrc/moe_kernels.cu). Here every rank is a thread (plus one "communication
// stream" thread per rank in the ZeRO model), the flags are std::atomic<int> used with exactly those memory orders, and
// the payloads (gradient slots, weight shards, token buffers) are PLAIN arrays. ThreadSanitizer tracks happens-before
// through the atomics, so an access that the flags do not order is reported as a data race even when the timing of
// the run happened to be harmless; the program itself checks the payload values (a stale or torn buffer) and
// returns 3. One rule at a time can be switched off on the command line to show that the model notices its absence.
//
//   protocol_model zero3 <world> <units> <steps> [drop]     drop: none | ready | consumed | version
//   protocol_model moe   <world> <calls>          [drop]     drop: none | dispatch | combine
//
// Build: g++ -O1 -g -std=c++17 -fsanitize=thread protocol_model.cpp -o protocol_model -lpthread
// The reference has no such protocol (its collectives are in-process stubs, ghostflow-nn/src/distributed.rs:147-207).
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr int PAYLOAD = 64;                  // ints per buffer: enough for TSAN to see the accesses
std::atomic<int> g_bad{0};                   // payload check failed (stale / torn data)
std::atomic<int> g_timeout{0};               // a bounded wait ran out

struct Flags {
  std::vector<std::unique_ptr<std::atomic<int>[]>> pad;   // [rank][index]
  Flags(int world, int n) {
    for (int r = 0; r < world; ++r) {
      pad.emplace_back(new std::atomic<int>[n]);
      for (int i = 0; i < n; ++i) pad.back()[i].store(0, std::memory_order_relaxed);
    }
  }
  // st.release.sys into the destination rank's pad
  void store(int dst, int idx, int v) { pad[dst][idx].store(v, std::memory_order_release); }
  // bounded ld.acquire poll of the owner
  bool wait_ge(int rank, int idx, int v) {
    const auto t0 = std::chrono::steady_clock::now();
    while (pad[rank][idx].load(std::memory_order_acquire) < v) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) {
        g_timeout.store(1);
        return false;
      }
      std::this_thread::yield();
    }
    return true;
  }
};

struct Buffer {
  int v[PAYLOAD];
  void fill(int tag) { for (int i = 0; i < PAYLOAD; ++i) v[i] = tag + i; }
  void expect(int tag) {
    for (int i = 0; i < PAYLOAD; ++i)
      if (v[i] != tag + i) { g_bad.store(1); return; }
  }
};

inline int tag_of(int kind, int unit, int step) { return kind * 1000000 + unit * 1000 + step * 100; }

// ------------------------------------------------------------------------------------------------- ZeRO-3
struct Task { int slot, unit, step, use; bool stop; };

struct Queue {
  std::mutex m;
  std::condition_variable cv;
  std::deque<Task> q;
  int done = 0;
  void push(Task t) { { std::lock_guard<std::mutex> l(m); q.push_back(t); } cv.notify_all(); }
  Task pop() { std::unique_lock<std::mutex> l(m); cv.wait(l, [&] { return !q.empty(); }); Task t = q.front(); q.pop_front(); return t; }
  void finished() { { std::lock_guard<std::mutex> l(m); ++done; } cv.notify_all(); }
  void wait_done(int n) { std::unique_lock<std::mutex> l(m); cv.wait(l, [&] { return done >= n; }); }
};

int run_zero3(int world, int units, int steps, const std::string& drop) {
  const bool wait_ready = drop != "ready", wait_consumed = drop != "consumed", wait_version = drop != "version";
  const int READY = 0, CONSUMED = 2 * world, VERSION = 4 * world;
  Flags flags(world, VERSION + units * world);
  std::vector<std::vector<Buffer>> shard(world, std::vector<Buffer>(units));   // weight shards
  std::vector<std::vector<Buffer>> grad(world, std::vector<Buffer>(2));        // two gradient slots per rank
  for (int r = 0; r < world; ++r)
    for (int u = 0; u < units; ++u) shard[r][u].fill(tag_of(1, u, 0));
  std::vector<Queue> queues(world);

  auto gather = [&](int r, int u, int version) {
    for (int o = 1; o <= world; ++o) {
      const int src = (r + o) % world;
      if (src != r && wait_version && !flags.wait_ge(r, VERSION + u * world + src, version)) return;
      if (src != r) shard[src][u].expect(tag_of(1, u, version));     // peer load of the shard
    }
  };
  auto reducer = [&](int r) {                                         // the rank's communication stream
    for (;;) {
      Task t = queues[r].pop();
      if (t.stop) return;
      bool ok = true;
      if (wait_ready)
        for (int src = 0; src < world && ok; ++src) ok = flags.wait_ge(r, READY + t.slot * world + src, t.use);
      if (ok) {
        for (int src = 0; src < world; ++src) grad[src][t.slot].expect(tag_of(2, t.unit, t.step));   // peer loads
        shard[r][t.unit].fill(tag_of(1, t.unit, t.step));                                        // AdamW on my shard
        for (int dst = 0; dst < world; ++dst) {
          flags.store(dst, CONSUMED + t.slot * world + r, t.use);
          flags.store(dst, VERSION + t.unit * world + r, t.step);
        }
      }
      queues[r].finished();
    }
  };
  auto compute = [&](int r) {
    int uses[2] = {0, 0}, submitted = 0;
    for (int t = 1; t <= steps; ++t) {
      for (int u = 0; u < units; ++u) gather(r, u, t - 1);            // forward
      int slot = 0;
      for (int u = units - 1; u >= 0; --u) {                          // backward
        if (wait_consumed && uses[slot])
          for (int src = 0; src < world; ++src)
            if (!flags.wait_ge(r, CONSUMED + slot * world + src, uses[slot])) return;
        grad[r][slot].fill(tag_of(2, u, t));
        ++uses[slot];
        for (int dst = 0; dst < world; ++dst) flags.store(dst, READY + slot * world + r, uses[slot]);
        queues[r].push(Task{slot, u, t, uses[slot], false});
        ++submitted;
        slot ^= 1;
      }
      queues[r].wait_done(submitted);                                 // end of step: join the communication stream
    }
    queues[r].push(Task{0, 0, 0, 0, true});
  };
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) {
    th.emplace_back(reducer, r);
    th.emplace_back(compute, r);
  }
  for (auto& t : th) t.join();
  return 0;
}

// ------------------------------------------------------------------------------------------------- MoE
int run_moe(int world, int calls, const std::string& drop) {
  const bool wait_dispatch = drop != "dispatch", wait_combine = drop != "combine";
  const int DISPATCH = 0, COMBINE = world;
  Flags flags(world, 2 * world);
  std::vector<std::vector<Buffer>> xs(world, std::vector<Buffer>(world));     // xs[owner][source]
  std::vector<std::vector<Buffer>> comb(world, std::vector<Buffer>(world));   // comb[source][owner]
  auto rank = [&](int r) {
    for (int e = 1; e <= calls; ++e) {
      for (int owner = 0; owner < world; ++owner) {                 // dispatch: rows into every owner's buffer
        xs[owner][r].fill(tag_of(3, r, e));
        flags.store(owner, DISPATCH + r, e);
      }
      if (wait_dispatch)
        for (int src = 0; src < world; ++src)
          if (!flags.wait_ge(r, DISPATCH + src, e)) return;
      for (int src = 0; src < world; ++src) xs[r][src].expect(tag_of(3, src, e));   // first expert GEMM reads
      for (int src = 0; src < world; ++src) {                      // second GEMM scatters the results home
        comb[src][r].fill(tag_of(4, r, e));
        flags.store(src, COMBINE + r, e);
      }
      if (wait_combine)
        for (int owner = 0; owner < world; ++owner)
          if (!flags.wait_ge(r, COMBINE + owner, e)) return;
      for (int owner = 0; owner < world; ++owner) comb[r][owner].expect(tag_of(4, owner, e));   // combine reads
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < world; ++r) th.emplace_back(rank, r);
  for (auto& t : th) t.join();
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 4) {
    fprintf(stderr, "usage: %s zero3 <world> <units> <steps> [drop] | moe <world> <calls> [drop]\n", argv[0]);
    return 2;
  }
  const std::string what = argv[1];
  if (what == "zero3" && argc >= 5)
    run_zero3(atoi(argv[2]), atoi(argv[3]), atoi(argv[4]), argc > 5 ? argv[5] : "none");
  else if (what == "moe")
    run_moe(atoi(argv[2]), atoi(argv[3]), argc > 4 ? argv[4] : "none");
  else
    return 2;
  if (g_timeout.load()) { fprintf(stderr, "a bounded wait ran out\n"); return 4; }
  if (g_bad.load()) { fprintf(stderr, "payload check failed: a buffer was read stale or torn\n"); return 3; }
  printf("ok\n");
  return 0;
}

// Stress test of the native runtime, meant to be built together with the runtime sources under a sanitizer
// (-fsanitize=thread, or -fsanitize=address,undefined) and run as a plain executable:
//
//   g++ -std=c++17 -g -O1 -fsanitize=thread -pthread cpp-package/tests/runtime_stress.cc \
//       mxnet_b200/csrc/engine.cc mxnet_b200/csrc/storage.cc -ldl -lrt -o runtime_stress && ./runtime_stress
//
// 1. Random dependency workloads (the scheme of tests/cpp/engine/threaded_engine_test.cc in the reference): a set of
//    integer cells, operations that read some cells and overwrite one, pushed to the engine with exactly those
//    read/write sets; the result must equal the serial evaluation for every engine kind and worker count.
// 2. Failure propagation: a failing operation poisons what it writes, dependants are skipped, unrelated work goes on,
//    the error surfaces at the wait and the engine stays usable.
// 3. The storage pool under concurrent allocation and release from several threads.
// Exit code 0 = all checks passed; each failed check prints a line and makes the exit code 1.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

extern "C" {
typedef int (*TaskFn)(void* arg, char* errbuf, int errlen);
void* mxb_engine_create(int naive, int nworkers);
void mxb_engine_destroy(void* e);
void* mxb_engine_new_var(void* e);
void mxb_engine_delete_var(void* e, void* v);
uint64_t mxb_engine_var_version(void* v);
void mxb_engine_push(void* e, TaskFn fn, void* arg, void** reads, int nr, void** writes, int nw, int priority, const char* name);
int mxb_engine_wait_var(void* e, void* v, char* err, int errlen);
int mxb_engine_wait_all(void* e, char* err, int errlen);
int64_t mxb_engine_num_pending(void* e);
void* mxb_pool_create(int dev_type, int dev_id, int strategy, uint64_t page, uint64_t large_round, int reserve_pct, int cutoff);
void mxb_pool_destroy(void* p);
void* mxb_pool_alloc(void* p, uint64_t nbytes, int failsafe, uint64_t* rounded);
void mxb_pool_free(void* p, void* ptr, uint64_t rounded);
void mxb_pool_release_all(void* p);
void mxb_pool_stats(void* p, int64_t* out6);
}

namespace {

int failures = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      std::printf("FAILED %s:%d: ", __FILE__, __LINE__);   \
      std::printf(__VA_ARGS__);                            \
      std::printf("\n");                                   \
      ++failures;                                          \
    }                                                      \
  } while (0)

struct Op {
  std::vector<int> reads;
  int write;
  int64_t add;
  std::vector<int64_t>* cells;     // plain memory: the engine's ordering is what keeps these accesses race free
};

int run_op(void* arg, char*, int) {
  Op* op = static_cast<Op*>(arg);
  int64_t s = op->add;
  for (int r : op->reads) s += (*op->cells)[r] * 3 % 1000003;
  (*op->cells)[op->write] = s % 1000003;
  return 0;
}

std::vector<Op> make_workload(int ncells, int nops, unsigned seed, std::vector<int64_t>* cells) {
  std::mt19937 rng(seed);
  std::vector<Op> ops(nops);
  for (auto& op : ops) {
    const int nr = rng() % 4;
    op.write = rng() % ncells;
    for (int i = 0; i < nr; ++i) {
      const int r = rng() % ncells;
      if (r != op.write) op.reads.push_back(r);          // a cell is either read or written by one operation
    }
    op.add = rng() % 1000;
    op.cells = cells;
  }
  return ops;
}

void random_workloads() {
  const int ncells = 24, nops = 3000;
  for (unsigned seed = 1; seed <= 3; ++seed) {
    std::vector<int64_t> expect(ncells, 1);
    {
      auto ops = make_workload(ncells, nops, seed, &expect);
      for (auto& op : ops) run_op(&op, nullptr, 0);
    }
    const int configs[][2] = {{1, 1}, {0, 1}, {0, 4}, {0, 8}};      // {naive, workers}
    for (auto& cfg : configs) {
      std::vector<int64_t> cells(ncells, 1);
      auto ops = make_workload(ncells, nops, seed, &cells);
      void* e = mxb_engine_create(cfg[0], cfg[1]);
      std::vector<void*> vars(ncells);
      for (auto& v : vars) v = mxb_engine_new_var(e);
      for (size_t i = 0; i < ops.size(); ++i) {
        std::vector<void*> r;
        for (int c : ops[i].reads) r.push_back(vars[c]);
        void* w = vars[ops[i].write];
        mxb_engine_push(e, run_op, &ops[i], r.data(), (int)r.size(), &w, 1, (int)(i % 3), "stress");
      }
      char err[256];
      CHECK(mxb_engine_wait_all(e, err, sizeof(err)) == 0, "wait_all reported %s", err);
      CHECK(mxb_engine_num_pending(e) == 0, "operations still pending");
      for (int c = 0; c < ncells; ++c)
        CHECK(cells[c] == expect[c], "seed %u naive=%d workers=%d cell %d: %lld != %lld", seed, cfg[0], cfg[1], c,
              (long long)cells[c], (long long)expect[c]);
      for (auto& v : vars) mxb_engine_delete_var(e, v);
      mxb_engine_wait_all(e, err, sizeof(err));
      mxb_engine_destroy(e);
    }
  }
}

int fail_op(void*, char* err, int errlen) {
  std::snprintf(err, errlen, "expected failure");
  return 1;
}
int count_op(void* arg, char*, int) {
  static_cast<std::atomic<int>*>(arg)->fetch_add(1);
  return 0;
}

void failure_propagation() {
  for (int naive = 0; naive <= 1; ++naive) {
    void* e = mxb_engine_create(naive, 4);
    void* a = mxb_engine_new_var(e);
    void* b = mxb_engine_new_var(e);
    void* c = mxb_engine_new_var(e);
    std::atomic<int> ran_dependant{0}, ran_other{0};
    mxb_engine_push(e, fail_op, nullptr, nullptr, 0, &a, 1, 0, "fails");
    mxb_engine_push(e, count_op, &ran_dependant, &a, 1, &b, 1, 0, "dependant");
    mxb_engine_push(e, count_op, &ran_other, nullptr, 0, &c, 1, 0, "unrelated");
    char err[256] = {0};
    CHECK(mxb_engine_wait_var(e, c, err, sizeof(err)) == 0, "unrelated var carries an error: %s", err);
    CHECK(mxb_engine_wait_var(e, b, err, sizeof(err)) != 0 && std::strstr(err, "expected failure") != nullptr,
          "dependant var has no error (naive=%d): '%s'", naive, err);
    CHECK(mxb_engine_wait_var(e, b, err, sizeof(err)) == 0, "a failure is reported by one wait only");
    CHECK(ran_dependant.load() == 0, "the dependant ran although its input failed");
    CHECK(ran_other.load() == 1, "the unrelated operation did not run");
    CHECK(mxb_engine_wait_all(e, err, sizeof(err)) == 0, "wait_all repeats a failure that a wait on a var has reported");
    // a failure that no wait on a var picks up is reported by wait_all, once
    mxb_engine_push(e, fail_op, nullptr, nullptr, 0, &a, 1, 0, "fails again");
    CHECK(mxb_engine_wait_all(e, err, sizeof(err)) != 0, "wait_all did not report the failure");
    CHECK(mxb_engine_wait_all(e, err, sizeof(err)) == 0, "wait_all reports the failure twice");
    std::atomic<int> after{0};
    mxb_engine_push(e, count_op, &after, nullptr, 0, &c, 1, 0, "after");
    CHECK(mxb_engine_wait_var(e, c, err, sizeof(err)) == 0 && after.load() == 1, "the engine is not usable after a failure");
    const uint64_t v0 = mxb_engine_var_version(c);
    mxb_engine_push(e, count_op, &after, nullptr, 0, &c, 1, 0, "bump");
    mxb_engine_wait_var(e, c, err, sizeof(err));
    CHECK(mxb_engine_var_version(c) == v0 + 1, "a write did not advance the version of its var");
    for (void* v : {a, b, c}) mxb_engine_delete_var(e, v);
    mxb_engine_wait_all(e, err, sizeof(err));
    mxb_engine_destroy(e);
  }
}

void pool_threads() {
  for (int strategy = 0; strategy <= 2; ++strategy) {          // naive, round, unpooled
    void* pool = mxb_pool_create(/*cpu*/ 1, 0, strategy, 4096, 2 << 20, 5, 24);
    std::atomic<int> bad{0};
    std::vector<std::thread> threads;
    for (int t = 0; t < 6; ++t)
      threads.emplace_back([&, t] {
        std::mt19937 rng(100 + t);
        std::vector<std::pair<void*, uint64_t>> held;
        for (int i = 0; i < 400; ++i) {
          if (held.size() > 8 || (rng() % 3 == 0 && !held.empty())) {
            auto [p, r] = held.back();
            held.pop_back();
            unsigned char* b = static_cast<unsigned char*>(p);
            if (b[0] != (unsigned char)t || b[r - 1] != (unsigned char)t) bad.fetch_add(1);     // nobody else wrote into it
            mxb_pool_free(pool, p, r);
          } else {
            const uint64_t n = 1 + rng() % 70000;
            uint64_t rounded = 0;
            void* p = mxb_pool_alloc(pool, n, 0, &rounded);
            if (p == nullptr || rounded < n) { bad.fetch_add(1); continue; }
            std::memset(p, t, rounded);
            held.push_back({p, rounded});
          }
        }
        for (auto& h : held) mxb_pool_free(pool, h.first, h.second);
      });
    for (auto& th : threads) th.join();
    CHECK(bad.load() == 0, "strategy %d: %d bad blocks", strategy, bad.load());
    int64_t stats[6] = {0};
    mxb_pool_stats(pool, stats);
    mxb_pool_release_all(pool);
    mxb_pool_destroy(pool);
  }
}

}  // namespace

int main() {
  random_workloads();
  failure_propagation();
  pool_threads();
  std::printf(failures == 0 ? "runtime_stress: all checks passed\n" : "runtime_stress: %d checks failed\n", failures);
  return failures == 0 ? 0 : 1;
}

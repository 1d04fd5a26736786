// Native dependency engine for host-side tasks.
//
// Contract kept from the reference (include/mxnet/engine.h:213-437, src/engine/threaded_engine.cc):
//  * a Var serialises writers against readers/writers and lets readers run concurrently;
//  * an operation lists the vars it reads and the vars it mutates and is dispatched once every
//    one of them has granted access; dispatch order among ready operations follows priority,
//    then submission order;
//  * a failing operation stores its error in the vars it mutates; operations that depend on a
//    failed var are skipped and pass the error on; WaitForVar / WaitForAll rethrow it, once;
//  * a naive mode runs everything inline in the pushing thread (deterministic debugging).
// What differs: GPU work is ordered by CUDA streams and events, so this engine only schedules host
// tasks (data pipeline stages, checkpoint writers, KVStore control messages, Python callbacks).
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <queue>
#include <string>
#include <thread>
#include <vector>

namespace mxb {

typedef int (*TaskFn)(void* arg, char* errbuf, int errlen);

struct Opr;

struct Var {
  std::mutex mu;
  int running_reads = 0;
  bool running_write = false;
  struct Waiter { Opr* opr; bool write; };
  std::deque<Waiter> queue;
  uint64_t version = 0;
  std::string error;          // non-empty: the last writer failed
  bool to_delete = false;
};

struct Opr {
  TaskFn fn;
  void* arg;
  std::vector<Var*> reads, writes;
  std::atomic<int> wait{0};
  int priority = 0;
  uint64_t seq = 0;
  std::string name;
  bool always = false;        // runs even when an input var carries an error (synchronisation markers)
};

struct OprOrder {
  bool operator()(const Opr* a, const Opr* b) const {
    if (a->priority != b->priority) return a->priority < b->priority;   // max-heap on priority
    return a->seq > b->seq;                                            // FIFO among equals
  }
};

class Engine {
 public:
  // nprio == 0: one pool of workers serves one priority queue (the pooled policy, src/engine/threaded_engine_pooled.cc).
  // nprio > 0: `nprio` further workers serve ONLY operations pushed with a positive priority, which have a queue of
  // their own, so urgent work (gradient exchange control, batch hand-over) never waits behind long ordinary tasks
  // that already occupy every ordinary worker (the high-priority CPU pool of src/engine/threaded_engine_perdevice.cc).
  Engine(bool naive, int nworkers, int nprio = 0) : naive_(naive), split_(nprio > 0) {
    if (!naive_) {
      for (int i = 0; i < nworkers; ++i) workers_.emplace_back([this] { WorkerLoop(&ready_); });
      for (int i = 0; i < nprio; ++i) workers_.emplace_back([this] { WorkerLoop(&urgent_); });
    }
  }
  ~Engine() {
    WaitAllNoThrow();
    {
      std::lock_guard<std::mutex> lk(qmu_);
      stop_ = true;
    }
    qcv_.notify_all();
    for (auto& t : workers_) t.join();
  }

  Var* NewVar() { return new Var(); }

  void DeleteVar(Var* v) {
    // deletion is itself a write so it runs after everything already queued on the var
    Push([](void*, char*, int) { return 0; }, nullptr, {}, {v}, 0, "DeleteVar", true);
  }

  void Push(TaskFn fn, void* arg, std::vector<Var*> reads, std::vector<Var*> writes, int priority,
            const char* name, bool delete_written = false, bool always = false) {
    Opr* op = new Opr();
    op->fn = fn; op->arg = arg; op->priority = priority; op->name = name ? name : "";
    op->always = always;
    op->reads = std::move(reads); op->writes = std::move(writes);
    op->seq = seq_.fetch_add(1);
    if (delete_written) for (Var* v : op->writes) v->to_delete = true;
    pending_.fetch_add(1);
    if (naive_) { Execute(op); return; }
    op->wait.store(static_cast<int>(op->reads.size() + op->writes.size()) + 1);
    for (Var* v : op->reads) {
      bool ready;
      {
        std::lock_guard<std::mutex> lk(v->mu);
        ready = !v->running_write && v->queue.empty();
        if (ready) ++v->running_reads; else v->queue.push_back({op, false});
      }
      if (ready) Grant(op);
    }
    for (Var* v : op->writes) {
      bool ready;
      {
        std::lock_guard<std::mutex> lk(v->mu);
        ready = !v->running_write && v->running_reads == 0 && v->queue.empty();
        if (ready) v->running_write = true; else v->queue.push_back({op, true});
      }
      if (ready) Grant(op);
    }
    Grant(op);   // the guard count
  }

  // returns 0 or copies the error of the var into err
  int WaitForVar(Var* v, char* err, int errlen) {
    if (!naive_) {
      struct Sync { std::mutex mu; std::condition_variable cv; bool done = false; } s;
      Push([](void* a, char*, int) {
             auto* s = static_cast<Sync*>(a);
             {
               // notify under the lock: the waiter owns the Sync object and may destroy it
               // as soon as it can re-acquire the mutex
               std::lock_guard<std::mutex> lk(s->mu);
               s->done = true;
               s->cv.notify_all();
             }
             return 0;
           }, &s, {v}, {}, 1 << 20, "WaitForVar", false, /*always=*/true);
      std::unique_lock<std::mutex> lk(s.mu);
      s.cv.wait(lk, [&] { return s.done; });
    }
    // A failure is reported once: the wait that raises it clears it from the var (later readers run again) and from
    // the engine-wide record that WaitForAll reports (src/engine/threaded_engine.h ThrowException does the same).
    std::string e;
    {
      std::lock_guard<std::mutex> lk(v->mu);
      e.swap(v->error);
    }
    if (e.empty()) return 0;
    {
      std::lock_guard<std::mutex> lk(emu_);
      if (first_error_ == e) first_error_.clear();
    }
    Copy(e, err, errlen);
    return 1;
  }

  int WaitForAll(char* err, int errlen) {
    WaitAllNoThrow();
    std::lock_guard<std::mutex> lk(emu_);
    if (!first_error_.empty()) {
      Copy(first_error_, err, errlen);
      first_error_.clear();
      return 1;
    }
    return 0;
  }

  int64_t NumPending() const { return pending_.load(); }

 private:
  static void Copy(const std::string& s, char* err, int errlen) {
    if (err && errlen > 0) {
      std::strncpy(err, s.c_str(), errlen - 1);
      err[errlen - 1] = 0;
    }
  }

  void WaitAllNoThrow() {
    std::unique_lock<std::mutex> lk(dmu_);
    dcv_.wait(lk, [this] { return pending_.load() == 0; });
  }

  void Grant(Opr* op) {
    if (op->wait.fetch_sub(1) == 1) {
      {
        std::lock_guard<std::mutex> lk(qmu_);
        (split_ && op->priority > 0 ? urgent_ : ready_).push(op);
      }
      qcv_.notify_all();
    }
  }

  using Queue = std::priority_queue<Opr*, std::vector<Opr*>, OprOrder>;

  void WorkerLoop(Queue* q) {
    for (;;) {
      Opr* op;
      {
        std::unique_lock<std::mutex> lk(qmu_);
        qcv_.wait(lk, [this, q] { return stop_ || !q->empty(); });
        if (stop_ && q->empty()) return;
        op = q->top();
        q->pop();
      }
      Execute(op);
    }
  }

  void Execute(Opr* op) {
    std::string err;
    for (Var* v : op->reads) {            // an upstream failure skips this operation
      std::lock_guard<std::mutex> lk(v->mu);
      if (!v->error.empty()) { err = v->error; break; }
    }
    if (op->always) {
      if (op->fn) op->fn(op->arg, nullptr, 0);
      err.clear();                        // a marker neither fails nor forwards a failure
    } else if (err.empty() && op->fn) {
      char buf[2048];
      buf[0] = 0;
      int rc = op->fn(op->arg, buf, sizeof(buf));
      if (rc != 0) err = buf[0] ? buf : ("operation " + op->name + " failed");
    }
    if (!err.empty()) {
      std::lock_guard<std::mutex> lk(emu_);
      if (first_error_.empty()) first_error_ = err;
    }
    for (Var* v : op->reads) CompleteRead(v);
    for (Var* v : op->writes) CompleteWrite(v, err);
    delete op;
    if (pending_.fetch_sub(1) == 1) {
      std::lock_guard<std::mutex> lk(dmu_);
      dcv_.notify_all();
    }
  }

  void CompleteRead(Var* v) {
    if (naive_) return;
    Opr* next = nullptr;
    {
      std::lock_guard<std::mutex> lk(v->mu);
      if (--v->running_reads == 0 && !v->queue.empty() && v->queue.front().write) {
        next = v->queue.front().opr;
        v->queue.pop_front();
        v->running_write = true;
      }
    }
    if (next) Grant(next);
  }

  void CompleteWrite(Var* v, const std::string& err) {
    std::vector<Opr*> grant;
    bool del = false;
    {
      std::lock_guard<std::mutex> lk(v->mu);
      v->running_write = false;
      ++v->version;
      v->error = err;                    // a successful write clears an older failure
      if (!naive_) {
        while (!v->queue.empty() && !v->queue.front().write) {
          grant.push_back(v->queue.front().opr);
          v->queue.pop_front();
          ++v->running_reads;
        }
        if (grant.empty() && !v->queue.empty()) {
          grant.push_back(v->queue.front().opr);
          v->queue.pop_front();
          v->running_write = true;
        }
      }
      del = v->to_delete && v->queue.empty() && v->running_reads == 0 && !v->running_write;
    }
    for (Opr* o : grant) Grant(o);
    if (del) delete v;
  }

  bool naive_;
  bool split_;
  std::vector<std::thread> workers_;
  std::priority_queue<Opr*, std::vector<Opr*>, OprOrder> ready_;
  std::priority_queue<Opr*, std::vector<Opr*>, OprOrder> urgent_;
  std::mutex qmu_;
  std::condition_variable qcv_;
  bool stop_ = false;
  std::atomic<int64_t> pending_{0};
  std::atomic<uint64_t> seq_{0};
  std::mutex dmu_;
  std::condition_variable dcv_;
  std::mutex emu_;
  std::string first_error_;
};

}  // namespace mxb

extern "C" {

void* mxb_engine_create(int naive, int nworkers) { return new mxb::Engine(naive != 0, nworkers < 1 ? 1 : nworkers); }
// kind: 0 = pooled (one queue, `nworkers` workers), 1 = naive (inline), 2 = ordinary pool + `nprio` workers that serve
// only positive-priority operations
void* mxb_engine_create_ex(int kind, int nworkers, int nprio) {
  if (kind == 1) return new mxb::Engine(true, 1);
  return new mxb::Engine(false, nworkers < 1 ? 1 : nworkers, kind == 2 ? (nprio < 1 ? 1 : nprio) : 0);
}
void mxb_engine_destroy(void* e) { delete static_cast<mxb::Engine*>(e); }
void* mxb_engine_new_var(void* e) { return static_cast<mxb::Engine*>(e)->NewVar(); }
void mxb_engine_delete_var(void* e, void* v) { static_cast<mxb::Engine*>(e)->DeleteVar(static_cast<mxb::Var*>(v)); }
uint64_t mxb_engine_var_version(void* v) {
  auto* var = static_cast<mxb::Var*>(v);
  std::lock_guard<std::mutex> lk(var->mu);
  return var->version;
}
void mxb_engine_push(void* e, mxb::TaskFn fn, void* arg, void** reads, int nr, void** writes, int nw, int priority,
                     const char* name) {
  std::vector<mxb::Var*> r(nr), w(nw);
  for (int i = 0; i < nr; ++i) r[i] = static_cast<mxb::Var*>(reads[i]);
  for (int i = 0; i < nw; ++i) w[i] = static_cast<mxb::Var*>(writes[i]);
  static_cast<mxb::Engine*>(e)->Push(fn, arg, std::move(r), std::move(w), priority, name);
}
int mxb_engine_wait_var(void* e, void* v, char* err, int errlen) {
  return static_cast<mxb::Engine*>(e)->WaitForVar(static_cast<mxb::Var*>(v), err, errlen);
}
int mxb_engine_wait_all(void* e, char* err, int errlen) { return static_cast<mxb::Engine*>(e)->WaitForAll(err, errlen); }
int64_t mxb_engine_num_pending(void* e) { return static_cast<mxb::Engine*>(e)->NumPending(); }

}  // extern "C"

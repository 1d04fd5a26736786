// Profiler back end: event store, Chrome trace-event JSON writer, aggregate statistics.
//
// Reference: src/profiler/profiler.{h,cc} (modes, "traceEvents" dump profiler.cc:183-250) and
// aggregate_stats.cc (per-name count/total/min/max/avg table).  Events carry the reference's
// categories ("operator", "api", "memory", user domains) so the emitted files open in
// chrome://tracing / Perfetto the same way.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace mxb {

struct Event {
  std::string name, cat;
  char ph;            // 'X' complete, 'B'/'E' begin/end, 'i' instant, 'C' counter
  int64_t ts, dur;
  int pid, tid;
  double value;
};

struct Profiler {
  std::mutex mu;
  std::vector<Event> events;
  bool running = false;
  bool aggregate = true;
  std::map<int, std::string> process_names;
};

static Profiler& P() { static Profiler p; return p; }

static std::string Escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if (c == '\n') o += "\\n";
    else o += c;
  }
  return o;
}

}  // namespace mxb

extern "C" {

int64_t mxb_prof_now_us() {
  using namespace std::chrono;
  return duration_cast<microseconds>(steady_clock::now().time_since_epoch()).count();
}
void mxb_prof_set_state(int running) { std::lock_guard<std::mutex> lk(mxb::P().mu); mxb::P().running = running != 0; }
int mxb_prof_get_state() { return mxb::P().running ? 1 : 0; }
void mxb_prof_clear() { std::lock_guard<std::mutex> lk(mxb::P().mu); mxb::P().events.clear(); }
void mxb_prof_name_process(int pid, const char* name) { std::lock_guard<std::mutex> lk(mxb::P().mu); mxb::P().process_names[pid] = name; }
void mxb_prof_add(const char* name, const char* cat, char ph, int64_t ts, int64_t dur, int pid, int tid, double value) {
  auto& p = mxb::P();
  std::lock_guard<std::mutex> lk(p.mu);
  if (!p.running) return;
  p.events.push_back({name, cat, ph, ts, dur, pid, tid, value});
}
int64_t mxb_prof_count() { std::lock_guard<std::mutex> lk(mxb::P().mu); return static_cast<int64_t>(mxb::P().events.size()); }

int mxb_prof_dump(const char* path) {
  auto& p = mxb::P();
  std::lock_guard<std::mutex> lk(p.mu);
  FILE* f = std::fopen(path, "w");
  if (!f) return 1;
  std::fprintf(f, "{\n    \"traceEvents\": [\n");
  bool first = true;
  for (auto& kv : p.process_names) {
    std::fprintf(f, "%s        {\"ph\": \"M\", \"args\": {\"name\": \"%s\"}, \"pid\": %d, \"name\": \"process_name\"}",
                 first ? "" : ",\n", mxb::Escape(kv.second).c_str(), kv.first);
    first = false;
  }
  for (auto& e : p.events) {
    std::fprintf(f, "%s        {\"name\": \"%s\", \"cat\": \"%s\", \"ph\": \"%c\", \"ts\": %lld, \"pid\": %d, \"tid\": %d",
                 first ? "" : ",\n", mxb::Escape(e.name).c_str(), mxb::Escape(e.cat).c_str(), e.ph,
                 static_cast<long long>(e.ts), e.pid, e.tid);
    if (e.ph == 'X') std::fprintf(f, ", \"dur\": %lld", static_cast<long long>(e.dur));
    if (e.ph == 'C') std::fprintf(f, ", \"args\": {\"%s\": %g}", mxb::Escape(e.name).c_str(), e.value);
    if (e.ph == 'i') std::fprintf(f, ", \"s\": \"p\"");
    std::fprintf(f, "}");
    first = false;
  }
  std::fprintf(f, "\n    ],\n    \"displayTimeUnit\": \"ms\"\n}\n");
  std::fclose(f);
  return 0;
}

// Aggregate statistics as text ("table") or JSON.  sort_by: 0 total, 1 avg, 2 min, 3 max, 4 count.
// Returns the number of bytes needed (including the terminator); writes at most cap bytes.
int64_t mxb_prof_aggregate(char* out, int64_t cap, int json, int sort_by, int ascending, int reset) {
  auto& p = mxb::P();
  std::lock_guard<std::mutex> lk(p.mu);
  struct Stat { int64_t count = 0, total = 0, mn = INT64_MAX, mx = 0; };
  std::map<std::string, std::map<std::string, Stat>> by_cat;
  std::map<std::string, std::vector<int64_t>> open;   // B/E pairing per (cat|name|tid)
  for (auto& e : p.events) {
    int64_t dur = -1;
    if (e.ph == 'X') dur = e.dur;
    else if (e.ph == 'B') open[e.cat + "|" + e.name + "|" + std::to_string(e.tid)].push_back(e.ts);
    else if (e.ph == 'E') {
      auto& st = open[e.cat + "|" + e.name + "|" + std::to_string(e.tid)];
      if (!st.empty()) { dur = e.ts - st.back(); st.pop_back(); }
    }
    if (dur < 0) continue;
    auto& s = by_cat[e.cat][e.name];
    ++s.count; s.total += dur; s.mn = std::min(s.mn, dur); s.mx = std::max(s.mx, dur);
  }
  std::ostringstream os;
  auto key = [sort_by](const Stat& s) -> double {
    switch (sort_by) { case 1: return s.count ? double(s.total) / s.count : 0; case 2: return double(s.mn);
                       case 3: return double(s.mx); case 4: return double(s.count); default: return double(s.total); }
  };
  if (json) os << "{\"Time\": {";
  else os << "\nProfile Statistics:\n\tNote the difference in units for different entries.\n";
  bool firstc = true;
  for (auto& c : by_cat) {
    std::vector<std::pair<std::string, Stat>> rows(c.second.begin(), c.second.end());
    std::sort(rows.begin(), rows.end(), [&](const std::pair<std::string, Stat>& a, const std::pair<std::string, Stat>& b) {
      return ascending ? key(a.second) < key(b.second) : key(a.second) > key(b.second);
    });
    if (json) {
      os << (firstc ? "" : ", ") << "\"" << mxb::Escape(c.first) << "\": {";
      bool firstr = true;
      for (auto& r : rows) {
        os << (firstr ? "" : ", ") << "\"" << mxb::Escape(r.first) << "\": {\"Count\": " << r.second.count
           << ", \"Total\": " << r.second.total / 1000.0 << ", \"Min\": " << r.second.mn / 1000.0
           << ", \"Max\": " << r.second.mx / 1000.0 << ", \"Avg\": " << (r.second.total / 1000.0) / r.second.count << "}";
        firstr = false;
      }
      os << "}";
    } else {
      char line[512];
      os << c.first << "\n=================\n";
      std::snprintf(line, sizeof(line), "%-40s %12s %16s %16s %16s %16s\n", "Name", "Total Count", "Time (ms)",
                    "Min Time (ms)", "Max Time (ms)", "Avg Time (ms)");
      os << line;
      std::snprintf(line, sizeof(line), "%-40s %12s %16s %16s %16s %16s\n", "----", "-----------", "---------",
                    "-------------", "-------------", "-------------");
      os << line;
      for (auto& r : rows) {
        std::snprintf(line, sizeof(line), "%-40s %12lld %16.4f %16.4f %16.4f %16.4f\n", r.first.c_str(),
                      static_cast<long long>(r.second.count), r.second.total / 1000.0, r.second.mn / 1000.0,
                      r.second.mx / 1000.0, (r.second.total / 1000.0) / r.second.count);
        os << line;
      }
      os << "\n";
    }
    firstc = false;
  }
  if (json) os << "}, \"Unit\": {\"Time\": \"ms\"}}";
  if (reset) p.events.clear();
  std::string s = os.str();
  if (out && cap > 0) {
    std::strncpy(out, s.c_str(), cap - 1);
    out[cap - 1] = 0;
  }
  return static_cast<int64_t>(s.size()) + 1;
}

}  // extern "C"

// A graph-pass library on the C ABI of mxb_lib_api.h: the pass "swap_op" rewrites every node whose operator is the
// option `from` into the operator `to` (same inputs and attributes), working on the JSON text of the graph.
// Build:   g++ -O2 -shared -fPIC -I<include dir> pass_lib.cc -o libpass_lib.so
// Use:     mx.library.load('/abs/path/libpass_lib.so');  sym.optimize_for('swap_op', **{'from': 'sigmoid', 'to': 'tanh'})
#include <cstring>
#include <string>

#include "mxb_lib_api.h"

namespace {

thread_local std::string result;
std::string last_error;

const char* option(const MXBAttrs* opts, const char* key) {
  for (int i = 0; i < opts->num; ++i)
    if (std::strcmp(opts->keys[i], key) == 0) return opts->vals[i];
  return nullptr;
}

int swap_op(const char* graph_json, const MXBAttrs* opts, const char** out_json) {
  const char* from = option(opts, "from");
  const char* to = option(opts, "to");
  if (from == nullptr || to == nullptr) {
    last_error = "swap_op needs the options from= and to=";
    return 1;
  }
  // operator names are JSON strings without escapes: match the exact member text, with either spacing after the colon
  result.assign(graph_json);
  for (const char* sep : {"\"op\": \"", "\"op\":\""}) {
    const std::string needle = std::string(sep) + from + "\"";
    const std::string repl = std::string(sep) + to + "\"";
    for (size_t pos = result.find(needle); pos != std::string::npos; pos = result.find(needle, pos + repl.size()))
      result.replace(pos, needle.size(), repl);
  }
  *out_json = result.c_str();
  return 0;
}

const MXBPassDesc kPasses[] = {{"swap_op", swap_op}};

}  // namespace

extern "C" {
int mxb_lib_api_version(void) { return MXB_LIB_API_VERSION; }
int mxb_lib_num_ops(void) { return 0; }
const MXBOpDesc* mxb_lib_op(int) { return nullptr; }
int mxb_lib_num_passes(void) { return 1; }
const MXBPassDesc* mxb_lib_pass(int index) { return &kPasses[index]; }
const char* mxb_lib_last_error(void) { return last_error.c_str(); }
}

// Lists the arrays of a .params file, scales every float32 array by 2 on the dependency engine (one task per array,
// all writing a shared counter variable in order), and writes the result to a second file.
//   g++ -std=c++17 -I cpp-package/include params_tool.cpp -L mxnet_b200/csrc -lmxb200_rt -o params_tool
#include <cstdio>
#include <mxb200/mxb200.hpp>

int main(int argc, char** argv) {
  if (argc < 3) { std::fprintf(stderr, "usage: params_tool in.params out.params\n"); return 2; }
  mxb200::ParamsFile in(argv[1]);
  mxb200::Engine engine(4);
  std::vector<std::vector<float>> scaled(in.arrays().size());
  auto done = engine.NewVar();
  int finished = 0;
  for (size_t i = 0; i < in.arrays().size(); ++i) {
    const mxb200::Array& a = in.arrays()[i];
    std::printf("%s ndim=%zu dtype=%d bytes=%llu\n", a.name.c_str(), a.shape.size(), a.dtype, (unsigned long long)a.nbytes);
    if (a.dtype != mxb200::kFloat32) continue;
    engine.Push([&, i] {
      const mxb200::Array& src = in.arrays()[i];
      const float* p = static_cast<const float*>(src.data);
      scaled[i].assign(p, p + src.nbytes / 4);
      for (float& v : scaled[i]) v *= 2.f;
      ++finished;                                   // serialised: every task writes `done`
    }, {}, {done});
  }
  engine.WaitForVar(done);
  mxb200::ParamsWriter out;
  for (size_t i = 0; i < in.arrays().size(); ++i) {
    const mxb200::Array& a = in.arrays()[i];
    if (a.dtype == mxb200::kFloat32) out.Add(a.name, a.shape, a.dtype, scaled[i].data(), a.nbytes);
    else out.Add(a.name, a.shape, a.dtype, a.data, a.nbytes);
  }
  out.Save(argv[2]);
  std::printf("tasks=%d\n", finished);
  // error propagation: a failing task surfaces at the wait
  auto v = engine.NewVar();
  engine.Push([] { throw std::runtime_error("expected failure"); }, {}, {v});
  try { engine.WaitForVar(v); return 1; } catch (const std::runtime_error& e) { std::printf("caught: %s\n", e.what()); }
  return 0;
}

// A multi-layer perceptron built and trained from C++ (the flow of cpp-package/example/mlp_cpu.cpp in the reference):
// symbols composed with Operator, arguments allocated by SimpleBind, Xavier initialisation, forward / backward through
// the Executor, SGD with momentum through the Optimizer, accuracy through the metric.  Data: 10 classes of 64-feature
// vectors around fixed random centres, generated here.
//
//   g++ -std=c++17 -O1 cpp-package/example/mlp_cpu.cpp -I cpp-package/include $(python3 -m pybind11 --includes) \
//       $(python3-config --ldflags --embed) -o mlp_cpu && PYTHONPATH=<repo>:<site-packages> ./mlp_cpu [gpu]
#include <cstdio>
#include <memory>
#include <random>

#include "mxb200/frontend.hpp"

using namespace mxb200;

static Symbol Mlp(const std::vector<int>& layers) {
  Symbol x = Symbol::Variable("X"), label = Symbol::Variable("label");
  Symbol out = x;
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string id = std::to_string(i);
    Symbol fc = Operator("FullyConnected")
                    .SetParam("num_hidden", layers[i])
                    .SetInput("data", out)
                    .SetInput("weight", Symbol::Variable("w" + id))
                    .SetInput("bias", Symbol::Variable("b" + id))
                    .CreateSymbol("fc" + id);
    out = i + 1 == layers.size() ? fc : Operator("Activation").SetParam("act_type", "relu").SetInput("data", fc).CreateSymbol("relu" + id);
  }
  return Operator("SoftmaxOutput").SetInput("data", out).SetInput("label", label).CreateSymbol("softmax");
}

int main(int argc, char** argv) {
  const Context ctx = argc > 1 && std::string(argv[1]) == "gpu" ? Context::gpu() : Context::cpu();
  const int features = 64, classes = 10, batch = 100, train_n = 2000, val_n = 500, epochs = 5;
  std::mt19937 rng(7);
  std::normal_distribution<float> noise(0.f, 0.6f);
  std::vector<float> centres(classes * features);
  for (auto& c : centres) c = noise(rng) * 2.f;
  auto make = [&](int n, std::vector<float>* xs, std::vector<float>* ys) {
    xs->resize((size_t)n * features);
    ys->resize(n);
    for (int i = 0; i < n; ++i) {
      const int c = rng() % classes;
      (*ys)[i] = (float)c;
      for (int f = 0; f < features; ++f) (*xs)[(size_t)i * features + f] = centres[c * features + f] + noise(rng);
    }
  };
  std::vector<float> tx, ty, vx, vy;
  make(train_n, &tx, &ty);
  make(val_n, &vx, &vy);

  Symbol net = Mlp({128, 64, classes});
  std::map<std::string, NDArray> args;
  args["X"] = NDArray(Shape(batch, features), ctx);
  args["label"] = NDArray(Shape(batch), ctx);
  std::unique_ptr<Executor> exe(net.SimpleBind(ctx, args));
  auto arg_dict = exe->arg_dict();
  Xavier xavier("gaussian", "in", 2.f);
  for (auto& kv : arg_dict) {
    if (kv.first == "X" || kv.first == "label") continue;
    if (kv.first[0] == 'w') xavier(kv.first, &kv.second); else kv.second = 0.f;
  }
  std::unique_ptr<Optimizer> opt(OptimizerRegistry::Find("sgd"));
  opt->SetParam("lr", 0.05)->SetParam("momentum", 0.9)->SetParam("rescale_grad", 1.0 / batch);
  const auto names = net.ListArguments();
  float acc = 0.f;
  for (int epoch = 0; epoch < epochs; ++epoch) {
    for (int start = 0; start + batch <= train_n; start += batch) {
      arg_dict["X"].SyncCopyFromCPU(tx.data() + (size_t)start * features, (size_t)batch * features);
      arg_dict["label"].SyncCopyFromCPU(ty.data() + start, batch);
      exe->Forward(true);
      exe->Backward();
      auto grads = exe->grad_dict();
      for (size_t i = 0; i < names.size(); ++i) {
        if (names[i] == "X" || names[i] == "label") continue;
        opt->Update((int)i, arg_dict[names[i]], grads[names[i]]);
      }
    }
    Accuracy metric;
    for (int start = 0; start + batch <= val_n; start += batch) {
      arg_dict["X"].SyncCopyFromCPU(vx.data() + (size_t)start * features, (size_t)batch * features);
      arg_dict["label"].SyncCopyFromCPU(vy.data() + start, batch);
      exe->Forward(false);
      metric.Update(arg_dict["label"], exe->outputs[0]);
    }
    acc = metric.Get();
    std::printf("epoch %d: validation accuracy %.3f\n", epoch, acc);
  }
  // imperative operators and file IO from C++
  NDArray a(std::vector<float>{1, -2, 3, -4}, Shape(2, 2), ctx);
  std::vector<NDArray> r = Operator("relu").PushInput(a).Invoke();
  NDArray::Save("mlp_cpu_weights.params", {{"arg:w0", arg_dict["w0"]}, {"relu", r[0]}});
  auto back = NDArray::LoadToMap("mlp_cpu_weights.params");
  std::printf("relu -> %.0f %.0f %.0f %.0f; saved %zu arrays; w0 %ux%u\n", r[0].At(0), r[0].At(1), r[0].At(2), r[0].At(3), back.size(),
              back["arg:w0"].GetShape()[0], back["arg:w0"].GetShape()[1]);
  NDArray::WaitAll();
  return acc > 0.9f ? 0 : 1;
}

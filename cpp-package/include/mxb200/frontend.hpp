// C++ front end for model code: NDArray, Symbol, Operator, Executor, Optimizer, KVStore, initializers, metrics, learning
// rate schedulers and data iterators with the call shapes of the reference's cpp-package (include/mxnet-cpp/*.h).
//
// The reference wraps libmxnet's C API.  Here the framework's front end is Python on top of the tensor library, so this
// header embeds the interpreter (pybind11) and forwards every call to the `mxnet_b200` package: a C++ program sees the
// same operators, kernels and file formats as a Python program, and tensors stay on their device between calls.
//
// Build:  g++ -std=c++17 prog.cpp -I cpp-package/include $(python3 -m pybind11 --includes) $(python3-config --ldflags --embed)
// Run:    PYTHONPATH must reach `mxnet_b200` and its dependencies (the site-packages of the environment it lives in).
#pragma once
#include <pybind11/embed.h>
#include <pybind11/numpy.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace mxb200 __attribute__((visibility("hidden"))) {
namespace py = pybind11;

typedef float mx_float;
typedef unsigned mx_uint;

// The interpreter and the imported package, started on first use and kept until the program ends.
class Runtime {
 public:
  static Runtime& Get() {
    static Runtime* rt = new Runtime();          // never destroyed: Python objects may outlive static destructors
    return *rt;
  }
  py::module_ mx, np;
  py::object nd, sym, autograd;

 private:
  Runtime() {
    if (!Py_IsInitialized()) guard_ = std::make_unique<py::scoped_interpreter>();
    mx = py::module_::import("mxnet_b200");
    np = py::module_::import("numpy");
    nd = mx.attr("nd");
    sym = mx.attr("sym");
    autograd = mx.attr("autograd");
  }
  std::unique_ptr<py::scoped_interpreter> guard_;
};

inline py::module_& MX() { return Runtime::Get().mx; }

enum DeviceType { kCPU = 1, kGPU = 2, kCPUPinned = 3 };

class Context {
 public:
  Context(DeviceType type, int id) : type_(type), id_(id) {}
  static Context cpu(int id = 0) { return Context(kCPU, id); }
  static Context gpu(int id = 0) { return Context(kGPU, id); }
  DeviceType GetDeviceType() const { return type_; }
  int GetDeviceId() const { return id_; }
  py::object py_ctx() const { return type_ == kGPU ? MX().attr("gpu")(id_) : (type_ == kCPUPinned ? MX().attr("cpu_pinned")(id_) : MX().attr("cpu")(id_)); }

 private:
  DeviceType type_;
  int id_;
};

class Shape {
 public:
  Shape() {}
  Shape(std::initializer_list<mx_uint> dims) : dims_(dims.begin(), dims.end()) {}
  explicit Shape(const std::vector<mx_uint>& dims) : dims_(dims) {}
  template <typename... Args>
  explicit Shape(mx_uint first, Args... rest) : dims_{first, static_cast<mx_uint>(rest)...} {}
  size_t ndim() const { return dims_.size(); }
  mx_uint operator[](size_t i) const { return dims_[i]; }
  size_t Size() const {
    size_t n = 1;
    for (mx_uint d : dims_) n *= d;
    return n;
  }
  const std::vector<mx_uint>& data() const { return dims_; }
  py::tuple py_tuple() const { return py::tuple(py::cast(dims_)); }

 private:
  std::vector<mx_uint> dims_;
};

class NDArray {
 public:
  NDArray() {}
  explicit NDArray(py::object handle) : h_(std::move(handle)) {}
  NDArray(const Shape& shape, const Context& ctx, bool /*delay_alloc*/ = true)
      : h_(Runtime::Get().nd.attr("zeros")(shape.py_tuple(), py::arg("ctx") = ctx.py_ctx())) {}
  NDArray(const std::vector<mx_float>& data, const Shape& shape, const Context& ctx) : NDArray(data.data(), shape, ctx) {}
  NDArray(const mx_float* data, const Shape& shape, const Context& ctx) {
    py::array_t<mx_float> a(shape.Size(), data);
    h_ = Runtime::Get().nd.attr("array")(a.attr("reshape")(shape.py_tuple()), py::arg("ctx") = ctx.py_ctx());
  }
  bool IsNone() const { return !h_ || h_.is_none(); }
  void SyncCopyFromCPU(const mx_float* data, size_t size) {
    py::array_t<mx_float> a(size, data);
    h_.attr("__setitem__")(py::slice(py::none(), py::none(), py::none()),
                           Runtime::Get().nd.attr("array")(a.attr("reshape")(h_.attr("shape")), py::arg("ctx") = h_.attr("context")));
  }
  void SyncCopyFromCPU(const std::vector<mx_float>& data) { SyncCopyFromCPU(data.data(), data.size()); }
  void SyncCopyToCPU(std::vector<mx_float>* out) const {
    py::array_t<mx_float> a = py::array_t<mx_float>::ensure(h_.attr("asnumpy")().attr("astype")("float32").attr("ravel")());
    out->assign(a.data(), a.data() + a.size());
  }
  std::vector<mx_float> ToVector() const {
    std::vector<mx_float> v;
    SyncCopyToCPU(&v);
    return v;
  }
  mx_float At(size_t flat_index) const { return ToVector().at(flat_index); }
  std::vector<mx_uint> GetShape() const { return h_.attr("shape").cast<std::vector<mx_uint>>(); }
  size_t Size() const { return h_.attr("size").cast<size_t>(); }
  Context GetContext() const {
    const bool gpu = h_.attr("context").attr("device_type").cast<std::string>() == "gpu";
    return Context(gpu ? kGPU : kCPU, h_.attr("context").attr("device_id").cast<int>());
  }
  NDArray Copy(const Context& ctx) const { return NDArray(h_.attr("copyto")(ctx.py_ctx())); }
  NDArray Slice(mx_uint begin, mx_uint end) const { return NDArray(h_.attr("__getitem__")(py::slice(begin, end, 1))); }
  NDArray Reshape(const Shape& shape) const { return NDArray(h_.attr("reshape")(shape.py_tuple())); }
  NDArray ArgmaxChannel() const { return NDArray(h_.attr("argmax")(py::arg("axis") = -1)); }
  void WaitToRead() const { h_.attr("wait_to_read")(); }
  void WaitToWrite() const { h_.attr("wait_to_read")(); }
  static void WaitAll() { Runtime::Get().nd.attr("waitall")(); }
  NDArray& operator=(mx_float scalar) {
    h_.attr("__setitem__")(py::slice(py::none(), py::none(), py::none()), scalar);
    return *this;
  }
  NDArray& operator+=(const NDArray& o) { h_ = h_.attr("__iadd__")(o.h_); return *this; }
  NDArray& operator-=(const NDArray& o) { h_ = h_.attr("__isub__")(o.h_); return *this; }
  NDArray& operator*=(mx_float s) { h_ = h_.attr("__imul__")(s); return *this; }
  NDArray& operator/=(mx_float s) { h_ = h_.attr("__itruediv__")(s); return *this; }
  friend NDArray operator+(const NDArray& a, const NDArray& b) { return NDArray(a.h_.attr("__add__")(b.h_)); }
  friend NDArray operator-(const NDArray& a, const NDArray& b) { return NDArray(a.h_.attr("__sub__")(b.h_)); }
  friend NDArray operator*(const NDArray& a, const NDArray& b) { return NDArray(a.h_.attr("__mul__")(b.h_)); }
  friend NDArray operator/(const NDArray& a, const NDArray& b) { return NDArray(a.h_.attr("__truediv__")(b.h_)); }
  friend NDArray operator+(const NDArray& a, mx_float s) { return NDArray(a.h_.attr("__add__")(s)); }
  friend NDArray operator-(const NDArray& a, mx_float s) { return NDArray(a.h_.attr("__sub__")(s)); }
  friend NDArray operator*(const NDArray& a, mx_float s) { return NDArray(a.h_.attr("__mul__")(s)); }
  friend NDArray operator/(const NDArray& a, mx_float s) { return NDArray(a.h_.attr("__truediv__")(s)); }
  static void Save(const std::string& file, const std::map<std::string, NDArray>& arrays) {
    py::dict d;
    for (auto& kv : arrays) d[py::str(kv.first)] = kv.second.h_;
    Runtime::Get().nd.attr("save")(file, d);
  }
  static std::map<std::string, NDArray> LoadToMap(const std::string& file) {
    std::map<std::string, NDArray> out;
    py::object loaded = Runtime::Get().nd.attr("load")(file);
    for (auto item : py::dict(loaded)) out[item.first.cast<std::string>()] = NDArray(py::reinterpret_borrow<py::object>(item.second));
    return out;
  }
  const py::object& handle() const { return h_; }

 private:
  py::object h_;
};

class Executor;

class Symbol {
 public:
  Symbol() {}
  explicit Symbol(py::object handle) : h_(std::move(handle)) {}
  explicit Symbol(const std::string& name) : h_(Runtime::Get().sym.attr("var")(name)) {}
  static Symbol Variable(const std::string& name) { return Symbol(name); }
  static Symbol Load(const std::string& file) { return Symbol(Runtime::Get().sym.attr("load")(file)); }
  static Symbol LoadJSON(const std::string& json) { return Symbol(Runtime::Get().sym.attr("load_json")(json)); }
  static Symbol Group(const std::vector<Symbol>& symbols) {
    py::list l;
    for (auto& s : symbols) l.append(s.h_);
    return Symbol(Runtime::Get().sym.attr("Group")(l));
  }
  void Save(const std::string& file) const { h_.attr("save")(file); }
  std::string ToJSON() const { return h_.attr("tojson")().cast<std::string>(); }
  std::string GetName() const { return h_.attr("name").is_none() ? std::string() : h_.attr("name").cast<std::string>(); }
  Symbol GetInternals() const { return Symbol(h_.attr("get_internals")()); }
  Symbol operator[](int index) const { return Symbol(h_.attr("__getitem__")(index)); }
  Symbol operator[](const std::string& name) const { return Symbol(h_.attr("__getitem__")(name)); }
  std::vector<std::string> ListArguments() const { return h_.attr("list_arguments")().cast<std::vector<std::string>>(); }
  std::vector<std::string> ListOutputs() const { return h_.attr("list_outputs")().cast<std::vector<std::string>>(); }
  std::vector<std::string> ListAuxiliaryStates() const { return h_.attr("list_auxiliary_states")().cast<std::vector<std::string>>(); }
  std::vector<std::string> ListInputs() const { return h_.attr("list_inputs")().cast<std::vector<std::string>>(); }
  // shapes of the arguments, outputs and auxiliary states given the shapes of some arguments
  void InferShape(const std::map<std::string, std::vector<mx_uint>>& known, std::vector<std::vector<mx_uint>>* arg_shapes,
                  std::vector<std::vector<mx_uint>>* aux_shapes, std::vector<std::vector<mx_uint>>* out_shapes) const {
    py::dict kw;
    for (auto& kv : known) kw[py::str(kv.first)] = py::tuple(py::cast(kv.second));
    py::tuple res = h_.attr("infer_shape")(**kw);
    auto conv = [](py::handle seq, std::vector<std::vector<mx_uint>>* out) {
      if (!out) return;
      out->clear();
      if (seq.is_none()) return;
      for (auto s : seq) out->push_back(s.is_none() ? std::vector<mx_uint>() : s.cast<std::vector<mx_uint>>());
    };
    conv(res[0], arg_shapes);
    conv(res[1], out_shapes);
    conv(res[2], aux_shapes);
  }
  // allocate every argument that is not given (shapes from inference) and bind
  inline Executor* SimpleBind(const Context& ctx, const std::map<std::string, NDArray>& args_map,
                              const std::map<std::string, NDArray>& arg_grad_store = {}, const std::string& grad_req = "write",
                              const std::map<std::string, NDArray>& aux_map = {});
  friend Symbol operator+(const Symbol& a, const Symbol& b) { return Symbol(a.h_.attr("__add__")(b.h_)); }
  friend Symbol operator-(const Symbol& a, const Symbol& b) { return Symbol(a.h_.attr("__sub__")(b.h_)); }
  friend Symbol operator*(const Symbol& a, const Symbol& b) { return Symbol(a.h_.attr("__mul__")(b.h_)); }
  friend Symbol operator/(const Symbol& a, const Symbol& b) { return Symbol(a.h_.attr("__truediv__")(b.h_)); }
  friend Symbol operator+(const Symbol& a, mx_float s) { return Symbol(a.h_.attr("__add__")(s)); }
  friend Symbol operator-(const Symbol& a, mx_float s) { return Symbol(a.h_.attr("__sub__")(s)); }
  friend Symbol operator*(const Symbol& a, mx_float s) { return Symbol(a.h_.attr("__mul__")(s)); }
  friend Symbol operator/(const Symbol& a, mx_float s) { return Symbol(a.h_.attr("__truediv__")(s)); }
  const py::object& handle() const { return h_; }

 private:
  py::object h_;
};

// Typed operator attributes for the generated wrappers of op.h: Attrs().Set("num_hidden", 64).Set("kernel", Shape(3, 3))
class Attrs {
 public:
  template <typename T>
  Attrs& Set(const std::string& key, const T& value) {
    d_[py::str(key)] = py::cast(value);
    return *this;
  }
  Attrs& Set(const std::string& key, const Shape& value) {
    d_[py::str(key)] = value.py_tuple();
    return *this;
  }
  Attrs& Set(const std::string& key, const char* value) {
    d_[py::str(key)] = py::str(value);
    return *this;
  }
  const py::dict& dict() const { return d_; }

 private:
  py::dict d_;
};

// Operator("FullyConnected").SetParam("num_hidden", 64).SetInput("data", x).CreateSymbol("fc1")
// Operator("relu").PushInput(array).Invoke()
class Operator {
 public:
  explicit Operator(const std::string& name) : name_(name) {}
  template <typename T>
  Operator& SetParam(const std::string& key, const T& value) {
    params_[py::str(key)] = py::cast(value);
    return *this;
  }
  Operator& SetParam(const std::string& key, const Shape& value) {
    params_[py::str(key)] = value.py_tuple();
    return *this;
  }
  Operator& SetParam(const std::string& key, const char* value) {
    params_[py::str(key)] = py::str(value);
    return *this;
  }
  Operator& SetAttrs(const Attrs& attrs) {
    for (auto item : attrs.dict()) params_[item.first] = item.second;
    return *this;
  }
  // an empty Symbol / NDArray (default constructed) stands for an optional input that is not given
  Operator& SetInput(const std::string& name, const Symbol& s) {
    if (s.handle()) named_[py::str(name)] = s.handle();
    return *this;
  }
  Operator& SetInput(const std::string& name, const NDArray& a) {
    if (a.handle()) named_[py::str(name)] = a.handle();
    return *this;
  }
  Operator& PushInput(const Symbol& s) { positional_.append(s.handle()); return *this; }
  Operator& PushInput(const NDArray& a) { positional_.append(a.handle()); return *this; }
  Operator& operator()() { return *this; }
  template <typename T, typename... Args>
  Operator& operator()(const T& first, const Args&... rest) {
    PushInput(first);
    return (*this)(rest...);
  }
  Symbol CreateSymbol(const std::string& name = "") {
    py::dict kw = Merge();
    if (!name.empty()) kw["name"] = py::str(name);
    return Symbol(Lookup(Runtime::Get().sym)(*py::tuple(positional_), **kw));
  }
  std::vector<NDArray> Invoke() {
    py::object res = Lookup(Runtime::Get().nd)(*py::tuple(positional_), **Merge());
    std::vector<NDArray> out;
    if (py::isinstance<py::list>(res) || py::isinstance<py::tuple>(res)) {
      for (auto r : res) out.emplace_back(py::reinterpret_borrow<py::object>(r));
    } else {
      out.emplace_back(res);
    }
    return out;
  }
  void Invoke(NDArray& output) {               // NOLINT: the reference's signature
    py::dict kw = Merge();
    kw["out"] = output.handle();
    Lookup(Runtime::Get().nd)(*py::tuple(positional_), **kw);
  }

 private:
  py::dict Merge() const {
    py::dict kw;
    for (auto item : params_) kw[item.first] = item.second;
    for (auto item : named_) kw[item.first] = item.second;
    return kw;
  }
  py::object Lookup(const py::object& ns) const {
    if (py::hasattr(ns, name_.c_str())) return ns.attr(name_.c_str());
    return ns.attr("op").attr(name_.c_str());    // names that start with an underscore live in the op module
  }
  std::string name_;
  py::dict params_, named_;
  py::list positional_;
};

class Executor {
 public:
  Executor(const Symbol& symbol, const Context& ctx, const std::map<std::string, NDArray>& args,
           const std::map<std::string, NDArray>& grads, const std::string& grad_req, const std::map<std::string, NDArray>& aux) {
    py::dict a, g, x;
    for (auto& kv : args) a[py::str(kv.first)] = kv.second.handle();
    for (auto& kv : grads) g[py::str(kv.first)] = kv.second.handle();
    for (auto& kv : aux) x[py::str(kv.first)] = kv.second.handle();
    h_ = symbol.handle().attr("_bind")(ctx.py_ctx(), a, py::arg("args_grad") = g.empty() ? py::object(py::none()) : py::object(g),
                                       py::arg("grad_req") = grad_req, py::arg("aux_states") = x.empty() ? py::object(py::none()) : py::object(x));
    Refresh();
  }
  void Forward(bool is_train) {
    h_.attr("forward")(py::arg("is_train") = is_train);
    outputs.clear();
    for (auto o : h_.attr("outputs")) outputs.emplace_back(py::reinterpret_borrow<py::object>(o));
  }
  void Backward(const std::vector<NDArray>& head_grads = {}) {
    if (head_grads.empty()) {
      h_.attr("backward")();
    } else {
      py::list l;
      for (auto& gq : head_grads) l.append(gq.handle());
      h_.attr("backward")(l);
    }
  }
  std::map<std::string, NDArray> arg_dict() const { return ToMap(h_.attr("arg_dict")); }
  std::map<std::string, NDArray> grad_dict() const { return ToMap(h_.attr("grad_dict")); }
  std::map<std::string, NDArray> aux_dict() const { return ToMap(h_.attr("aux_dict")); }
  std::vector<NDArray> outputs, arg_arrays, grad_arrays, aux_arrays;

 private:
  static std::map<std::string, NDArray> ToMap(const py::object& d) {
    std::map<std::string, NDArray> out;
    for (auto item : py::dict(d))
      if (!item.second.is_none()) out[item.first.cast<std::string>()] = NDArray(py::reinterpret_borrow<py::object>(item.second));
    return out;
  }
  void Refresh() {
    for (auto a : h_.attr("arg_arrays")) arg_arrays.emplace_back(py::reinterpret_borrow<py::object>(a));
    for (auto a : h_.attr("grad_arrays")) grad_arrays.emplace_back(a.is_none() ? py::object(py::none()) : py::reinterpret_borrow<py::object>(a));
    for (auto a : h_.attr("aux_arrays")) aux_arrays.emplace_back(py::reinterpret_borrow<py::object>(a));
  }
  py::object h_;
};

inline Executor* Symbol::SimpleBind(const Context& ctx, const std::map<std::string, NDArray>& args_map,
                                    const std::map<std::string, NDArray>& arg_grad_store, const std::string& grad_req,
                                    const std::map<std::string, NDArray>& aux_map) {
  std::map<std::string, std::vector<mx_uint>> known;
  for (auto& kv : args_map) known[kv.first] = kv.second.GetShape();
  std::vector<std::vector<mx_uint>> arg_shapes, aux_shapes, out_shapes;
  InferShape(known, &arg_shapes, &aux_shapes, &out_shapes);
  std::map<std::string, NDArray> args = args_map, grads = arg_grad_store, aux = aux_map;
  const auto arg_names = ListArguments();
  for (size_t i = 0; i < arg_names.size(); ++i) {
    if (!args.count(arg_names[i])) args[arg_names[i]] = NDArray(Shape(arg_shapes.at(i)), ctx);
    if (grad_req != "null" && !grads.count(arg_names[i])) grads[arg_names[i]] = NDArray(Shape(arg_shapes.at(i)), ctx);
  }
  const auto aux_names = ListAuxiliaryStates();
  for (size_t i = 0; i < aux_names.size(); ++i)
    if (!aux.count(aux_names[i])) aux[aux_names[i]] = NDArray(Shape(aux_shapes.at(i)), ctx);
  return new Executor(*this, ctx, args, grads, grad_req, aux);
}

// OptimizerRegistry::Find("sgd")->SetParam("lr", 0.1)->SetParam("momentum", 0.9); opt->Update(index, weight, grad)
class Optimizer {
 public:
  explicit Optimizer(const std::string& name) : name_(name) {}
  template <typename T>
  Optimizer* SetParam(const std::string& key, const T& value) {
    params_[py::str(key == "lr" ? "learning_rate" : key)] = py::cast(value);
    updater_ = py::none();
    return this;
  }
  void Update(int index, NDArray weight, NDArray grad) {
    if (!updater_ || updater_.is_none()) {
      py::object opt = MX().attr("optimizer").attr("create")(name_, **params_);
      updater_ = MX().attr("optimizer").attr("get_updater")(opt);
    }
    updater_(index, grad.handle(), weight.handle());
  }

 private:
  std::string name_;
  py::dict params_;
  py::object updater_;
};

class OptimizerRegistry {
 public:
  static Optimizer* Find(const std::string& name) { return new Optimizer(name); }
};

class KVStore {
 public:
  static void SetType(const std::string& type) { Store() = MX().attr("kv").attr("create")(type); }
  static void Init(int key, const NDArray& value) { Get().attr("init")(key, value.handle()); }
  static void Push(int key, const NDArray& value, int priority = 0) { Get().attr("push")(key, value.handle(), py::arg("priority") = priority); }
  static void Pull(int key, NDArray* out, int priority = 0) { Get().attr("pull")(key, py::arg("out") = out->handle(), py::arg("priority") = priority); }
  static std::string GetType() { return Get().attr("type").cast<std::string>(); }
  static int GetRank() { return Get().attr("rank").cast<int>(); }
  static int GetNumWorkers() { return Get().attr("num_workers").cast<int>(); }
  static void Barrier() { Get().attr("barrier")(); }

 private:
  static py::object& Store() {
    static py::object* s = new py::object();
    return *s;
  }
  static py::object& Get() {
    if (!Store()) SetType("local");
    return Store();
  }
};

class Initializer {
 public:
  virtual ~Initializer() {}
  // Names with the usual suffixes (weight, bias, gamma, beta, moving_*) get the pattern-based default of the Python
  // initializers; any other name receives the distribution itself.
  virtual void operator()(const std::string& name, NDArray* arr) {
    py::object desc = MX().attr("init").attr("InitDesc")(name);
    py::object init = Make();
    try {
      init(desc, arr->handle());
    } catch (py::error_already_set& e) {
      if (!e.matches(PyExc_ValueError)) throw;
      init.attr("_init_weight")(desc, arr->handle());
    }
  }

 protected:
  virtual py::object Make() = 0;
};
class Uniform : public Initializer {
 public:
  explicit Uniform(float scale = 0.07f) : scale_(scale) {}
 protected:
  py::object Make() override { return MX().attr("init").attr("Uniform")(scale_); }
  float scale_;
};
class Normal : public Initializer {
 public:
  explicit Normal(float sigma = 0.01f) : sigma_(sigma) {}
 protected:
  py::object Make() override { return MX().attr("init").attr("Normal")(sigma_); }
  float sigma_;
};
class Xavier : public Initializer {
 public:
  explicit Xavier(const std::string& rnd_type = "uniform", const std::string& factor_type = "avg", float magnitude = 3.f)
      : rnd_(rnd_type), factor_(factor_type), magnitude_(magnitude) {}
 protected:
  py::object Make() override {
    return MX().attr("init").attr("Xavier")(py::arg("rnd_type") = rnd_, py::arg("factor_type") = factor_, py::arg("magnitude") = magnitude_);
  }
  std::string rnd_, factor_;
  float magnitude_;
};

class EvalMetric {
 public:
  explicit EvalMetric(const std::string& name) : h_(MX().attr("gluon").attr("metric").attr("create")(name)) {}
  void Update(const NDArray& labels, const NDArray& preds) {
    py::list l, p;
    l.append(labels.handle());
    p.append(preds.handle());
    h_.attr("update")(l, p);
  }
  void Reset() { h_.attr("reset")(); }
  float Get() const { return py::tuple(h_.attr("get")())[1].cast<float>(); }

 private:
  py::object h_;
};
class Accuracy : public EvalMetric { public: Accuracy() : EvalMetric("acc") {} };
class LogLoss : public EvalMetric { public: LogLoss() : EvalMetric("ce") {} };
class MAE : public EvalMetric { public: MAE() : EvalMetric("mae") {} };
class MSE : public EvalMetric { public: MSE() : EvalMetric("mse") {} };
class RMSE : public EvalMetric { public: RMSE() : EvalMetric("rmse") {} };

class LRScheduler {
 public:
  explicit LRScheduler(py::object h) : h_(std::move(h)) {}
  float GetLR(unsigned num_update) { return h_(num_update).cast<float>(); }
 protected:
  py::object h_;
};
class FactorScheduler : public LRScheduler {
 public:
  FactorScheduler(int step, float factor = 1.f, float stop_factor_lr = 1e-8f, float base_lr = 0.01f)
      : LRScheduler(MX().attr("lr_scheduler").attr("FactorScheduler")(py::arg("step") = step, py::arg("factor") = factor,
                                                                     py::arg("stop_factor_lr") = stop_factor_lr, py::arg("base_lr") = base_lr)) {}
};

// MXDataIter("CSVIter").SetParam("data_csv", path).SetParam("batch_size", 32).CreateDataIter()
class MXDataIter {
 public:
  explicit MXDataIter(const std::string& type) : type_(type) {}
  template <typename T>
  MXDataIter& SetParam(const std::string& key, const T& value) {
    params_[py::str(key)] = py::cast(value);
    return *this;
  }
  MXDataIter& SetParam(const std::string& key, const Shape& value) {
    params_[py::str(key)] = value.py_tuple();
    return *this;
  }
  MXDataIter& CreateDataIter() {
    h_ = MX().attr("io").attr(type_.c_str())(**params_);
    return *this;
  }
  void Reset() { h_.attr("reset")(); }
  bool Next() {
    try {
      batch_ = h_.attr("next")();
      return true;
    } catch (py::error_already_set& e) {
      if (e.matches(PyExc_StopIteration)) return false;
      throw;
    }
  }
  NDArray GetData() const { return NDArray(py::reinterpret_borrow<py::object>(py::list(batch_.attr("data"))[0])); }
  NDArray GetLabel() const { return NDArray(py::reinterpret_borrow<py::object>(py::list(batch_.attr("label"))[0])); }
  int GetPadNum() const { return batch_.attr("pad").is_none() ? 0 : batch_.attr("pad").cast<int>(); }

 private:
  std::string type_;
  py::dict params_;
  py::object h_, batch_;
};

}  // namespace mxb200

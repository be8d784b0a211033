// Native CPU tensor + reverse-mode autograd core (f32), the host-side counterpart of the device kernels.
//
//   ft::TensorImpl   shape / strides / offset over shared storage, requires_grad, grad, grad_fn, hooks, version counter
//   ft::Node         one differentiable operation: the inputs it has to send gradients to and its backward rule
//   ft::backward     graph collection (breadth first from the root), dependency counts, Kahn ordering, reverse sweep; gradient contributions
//                    are kept per consuming edge and summed in edge order when a node becomes ready, so the serial engine and the parallel one
//                    (worker threads over the ready queue) give identical bits; tensor hooks (may rewrite a gradient) run before accumulation
//                    into a leaf, post-accumulate hooks after it (what DDP uses to launch a bucket's all-reduce)
//   operations       add / sub / mul / div (the second operand may have the shape of the trailing dimensions), scale, matmul, transpose, reshape, relu, tanh, sigmoid and the
//                    element-wise family (exp, log, sqrt, gelu, silu, leaky relu, power, abs, square, reciprocal), sum / mean over everything or
//                    along one dimension, softmax / log-softmax, linear, batched matmul, permute, narrow, layer norm, embedding, conv2d (patch matrix x GEMM),
//                    max_pool2d, cross-entropy on logits
//   ft::Sgd, ft::Adam momentum / dampening / nesterov / weight decay; Adam and AdamW (decoupled decay): same update rules as the device kernels
//
// Everything is exported through a small C ABI (opaque handles) for the Python binding in ferrotorch_b200/native.py.
//
// Capability parity: ferrotorch-core/src/tensor.rs:46-103 (GradFn, TensorInner), autograd/graph.rs:20-206 (backward: BFS + Kahn + reverse sweep
// + hooks), :220-458 (backward_parallel), grad_fns/{arithmetic,linalg,activation,reduction}.rs, ferrotorch-nn/src/{linear,loss}.rs,
// ferrotorch-optim/src/sgd.rs:30-210.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#define FT_API extern "C" __attribute__((visibility("default")))

namespace ft {

struct Node;
struct TensorImpl;
using Tensor = std::shared_ptr<TensorImpl>;

static std::atomic<uint64_t> g_next_id{1};
static thread_local bool g_grad_enabled = true;
static thread_local std::string g_last_error;

struct TensorImpl {
  std::shared_ptr<std::vector<float>> storage;
  std::vector<int64_t> shape, strides;
  int64_t offset = 0;
  bool requires_grad = false;
  Tensor grad;
  std::shared_ptr<Node> grad_fn;
  std::vector<std::function<void(TensorImpl&)>> hooks;             // run on the incoming gradient of this tensor (may modify it)
  std::vector<std::function<void(TensorImpl&)>> post_acc_hooks;    // run on a leaf after its .grad was updated
  uint64_t id = g_next_id++;
  uint32_t version = 0;

  int64_t numel() const { int64_t n = 1; for (auto s : shape) n *= s; return n; }
  bool is_leaf() const { return grad_fn == nullptr; }
  bool is_contiguous() const {
    int64_t expect = 1;
    for (int i = (int)shape.size() - 1; i >= 0; i--) {
      if (shape[i] != 1 && strides[i] != expect) return false;
      expect *= shape[i];
    }
    return true;
  }
  float* data() { return storage->data() + offset; }
  const float* data() const { return storage->data() + offset; }
};

static std::vector<int64_t> row_major(const std::vector<int64_t>& shape) {
  std::vector<int64_t> st(shape.size());
  int64_t s = 1;
  for (int i = (int)shape.size() - 1; i >= 0; i--) { st[i] = s; s *= shape[i]; }
  return st;
}
static Tensor make(const std::vector<int64_t>& shape, float fill = 0.f) {
  auto t = std::make_shared<TensorImpl>();
  t->shape = shape;
  t->strides = row_major(shape);
  t->storage = std::make_shared<std::vector<float>>((size_t)t->numel(), fill);
  return t;
}
static Tensor contiguous(const Tensor& a) {
  if (a->is_contiguous()) return a;
  Tensor o = make(a->shape);
  const int nd = (int)a->shape.size();
  std::vector<int64_t> idx(nd, 0);
  const int64_t n = a->numel();
  float* d = o->data();
  const float* s = a->data();
  for (int64_t i = 0; i < n; i++) {
    int64_t off = 0;
    for (int k = 0; k < nd; k++) off += idx[k] * a->strides[k];
    d[i] = s[off];
    for (int k = nd - 1; k >= 0; k--) { if (++idx[k] < a->shape[k]) break; idx[k] = 0; }
  }
  return o;
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// graph
// ---------------------------------------------------------------------------------------------------------------------------------------
struct Node {
  std::vector<Tensor> inputs;                       // null where the input needs no gradient
  const char* name = "node";
  virtual ~Node() = default;
  virtual std::vector<Tensor> backward(const Tensor& grad_out) = 0;   // one gradient per input (null allowed)
};

static bool needs_grad(std::initializer_list<Tensor> ts) {
  if (!g_grad_enabled) return false;
  for (auto& t : ts) if (t && t->requires_grad) return true;
  return false;
}
template <typename N, typename... A>
static void attach(const Tensor& out, std::initializer_list<Tensor> ins, A&&... args) {
  if (!needs_grad(ins)) return;
  auto n = std::make_shared<N>(std::forward<A>(args)...);
  for (auto& t : ins) n->inputs.push_back(t && t->requires_grad ? t : nullptr);
  out->requires_grad = true;
  out->grad_fn = n;
}

static void accumulate(Tensor& dst, const Tensor& src) {
  if (!dst) { dst = contiguous(src); if (dst.get() == src.get()) { dst = make(src->shape); std::memcpy(dst->data(), src->data(), sizeof(float) * (size_t)src->numel()); } return; }
  Tensor s = contiguous(src);
  float* d = dst->data();
  const float* p = s->data();
  const int64_t n = dst->numel();
  for (int64_t i = 0; i < n; i++) d[i] += p[i];
}

struct Engine {
  // per node (and per leaf): the slots of its incoming contributions (one per consuming edge, in discovery order) and how many are still missing
  struct Info { std::vector<Tensor> slots; int missing = 0; std::mutex mu; };
  std::unordered_map<Node*, std::unique_ptr<Info>> info;
  std::unordered_map<TensorImpl*, std::unique_ptr<Info>> leaf_info;
  std::unordered_map<Node*, std::shared_ptr<Node>> keep;
  std::unordered_map<const void*, int> slot_of;      // address of a consumer's input entry -> its slot in the producer (node or leaf)

  void collect(const std::shared_ptr<Node>& root) {
    std::deque<std::shared_ptr<Node>> q{root};
    keep[root.get()] = root;
    info[root.get()] = std::make_unique<Info>();
    while (!q.empty()) {
      auto n = q.front();
      q.pop_front();
      for (size_t i = 0; i < n->inputs.size(); i++) {
        const Tensor& t = n->inputs[i];
        if (!t) continue;
        Info* pi;
        if (t->grad_fn) {
          Node* p = t->grad_fn.get();
          if (!info.count(p)) { info[p] = std::make_unique<Info>(); keep[p] = t->grad_fn; q.push_back(t->grad_fn); }
          pi = info[p].get();
        } else {
          if (!leaf_info.count(t.get())) leaf_info[t.get()] = std::make_unique<Info>();
          pi = leaf_info[t.get()].get();
        }
        slot_of[&n->inputs[i]] = (int)pi->slots.size();
        pi->slots.emplace_back();
        pi->missing++;
      }
    }
  }
  static Tensor sum_slots(Info& in) {
    Tensor g;
    for (auto& s : in.slots) if (s) accumulate(g, s);      // edge order: the same sum whatever order the contributions arrived in
    return g;
  }
  // run one node: returns the producers that became ready
  std::vector<Node*> run(Node* n) {
    Info& in = *info.at(n);
    Tensor g = sum_slots(in);
    in.slots.clear();
    std::vector<Node*> ready;
    std::vector<Tensor> gi;
    if (g) gi = n->backward(g);
    for (size_t i = 0; i < n->inputs.size(); i++) {
      Tensor& t = n->inputs[i];
      if (!t) continue;
      Tensor gin = i < gi.size() ? gi[i] : nullptr;
      if (gin && !t->hooks.empty()) {
        Tensor c = make(gin->shape);                        // hooks may rewrite the gradient: give them a private copy
        Tensor gc = contiguous(gin);
        std::memcpy(c->data(), gc->data(), sizeof(float) * (size_t)gc->numel());
        gin = c;
        for (auto& h : t->hooks) h(*gin);
      }
      Info& pi = t->grad_fn ? *info.at(t->grad_fn.get()) : *leaf_info.at(t.get());
      bool now_ready;
      {
        std::lock_guard<std::mutex> lk(pi.mu);
        pi.slots[slot_of.at(&t)] = gin;
        now_ready = --pi.missing == 0;
      }
      if (!now_ready) continue;
      if (t->grad_fn) {
        ready.push_back(t->grad_fn.get());
      } else {
        // every consumer of this leaf has delivered: its gradient is final for this sweep
        Tensor total = sum_slots(pi);
        pi.slots.clear();
        if (total) {
          accumulate(t->grad, total);
          for (auto& h : t->post_acc_hooks) h(*t);
        }
      }
    }
    return ready;
  }
};

static void backward(const Tensor& root, const Tensor& grad_root, int threads) {
  if (!root->grad_fn) {
    if (root->requires_grad) { accumulate(root->grad, grad_root); for (auto& h : root->post_acc_hooks) h(*root); }
    return;
  }
  Engine e;
  e.collect(root->grad_fn);
  Engine::Info& ri = *e.info.at(root->grad_fn.get());
  ri.slots.push_back(grad_root);
  if (threads <= 1) {
    // Kahn: a node runs once every consumer has delivered its contribution; the ready list is a FIFO, so the order is a fixed function of the graph
    std::deque<Node*> ready{root->grad_fn.get()};
    while (!ready.empty()) {
      Node* n = ready.front();
      ready.pop_front();
      for (Node* p : e.run(n)) ready.push_back(p);
    }
    return;
  }
  std::mutex mu;
  std::condition_variable cv;
  std::deque<Node*> ready{root->grad_fn.get()};
  int running = 0;
  auto worker = [&] {
    std::unique_lock<std::mutex> lk(mu);
    while (true) {
      cv.wait(lk, [&] { return !ready.empty() || (running == 0); });
      if (ready.empty()) { if (running == 0) { cv.notify_all(); return; } continue; }
      Node* n = ready.front();
      ready.pop_front();
      running++;
      lk.unlock();
      std::vector<Node*> next = e.run(n);
      lk.lock();
      running--;
      for (Node* p : next) ready.push_back(p);
      cv.notify_all();
    }
  };
  std::vector<std::thread> pool;
  for (int i = 0; i < threads; i++) pool.emplace_back(worker);
  for (auto& t : pool) t.join();
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// operations (inputs are made contiguous; row-broadcast means b has the shape of a's last dimension)
// ---------------------------------------------------------------------------------------------------------------------------------------
// b may have the shape of a, or of a's trailing dimensions (a bias vector, a [S, S] mask under [B, H, S, S]): element i of a pairs with i % numel(b)
static bool suffix_broadcast_ok(const std::vector<int64_t>& a, const std::vector<int64_t>& b) {
  int64_t na = 1, nb0 = 1;
  for (auto v : a) na *= v;
  for (auto v : b) nb0 *= v;
  if (na == nb0 && na > 0) return true;                      // same number of elements: paired in order (a scalar with a one-element vector)
  if (b.size() > a.size() || b.empty()) return false;
  for (size_t i = 0; i < b.size(); i++)
    if (b[b.size() - 1 - i] != a[a.size() - 1 - i]) return false;
  int64_t nb = 1;
  for (auto v : b) nb *= v;
  return nb > 0;
}
static Tensor reduce_to(const Tensor& g, const std::vector<int64_t>& shape) {       // sum a [rows, n] gradient down to [n]
  if (g->shape == shape) return g;
  Tensor o = make(shape);
  const int64_t n = o->numel(), rows = g->numel() / n;
  Tensor gc = contiguous(g);
  for (int64_t r = 0; r < rows; r++) for (int64_t i = 0; i < n; i++) o->data()[i] += gc->data()[r * n + i];
  return o;
}
enum class Bin { Add, Sub, Mul };
struct BinNode : Node {
  Bin op; Tensor a, b;
  BinNode(Bin o, Tensor x, Tensor y) : op(o), a(std::move(x)), b(std::move(y)) { name = "binary"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), ga, gb;
    const int64_t n = gc->numel(), nb = b->numel();
    if (op == Bin::Mul) {
      ga = make(a->shape); gb = make(a->shape);
      for (int64_t i = 0; i < n; i++) { ga->data()[i] = gc->data()[i] * b->data()[i % nb]; gb->data()[i] = gc->data()[i] * a->data()[i]; }
    } else {
      ga = gc;
      gb = gc;
      if (op == Bin::Sub) { gb = make(a->shape); for (int64_t i = 0; i < n; i++) gb->data()[i] = -gc->data()[i]; }
    }
    return {ga, reduce_to(gb, b->shape)};
  }
};
static Tensor binary(Bin op, const Tensor& a0, const Tensor& b0) {
  Tensor a = contiguous(a0), b = contiguous(b0);
  const int64_t n = a->numel(), nb = b->numel();
  if (!suffix_broadcast_ok(a->shape, b->shape)) { g_last_error = "binary: shapes do not match or broadcast (the second operand must have the shape of the first or of its trailing dimensions)"; return nullptr; }
  Tensor o = make(a->shape);
  for (int64_t i = 0; i < n; i++) {
    const float x = a->data()[i], y = b->data()[i % nb];
    o->data()[i] = op == Bin::Add ? x + y : (op == Bin::Sub ? x - y : x * y);
  }
  attach<BinNode>(o, {a0, b0}, op, a, b);
  return o;
}
struct ScaleNode : Node {
  float s;
  explicit ScaleNode(float v) : s(v) { name = "scale"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(gc->shape);
    for (int64_t i = 0; i < gc->numel(); i++) o->data()[i] = gc->data()[i] * s;
    return {o};
  }
};
static Tensor scale(const Tensor& a0, float s) {
  Tensor a = contiguous(a0), o = make(a->shape);
  for (int64_t i = 0; i < a->numel(); i++) o->data()[i] = a->data()[i] * s;
  attach<ScaleNode>(o, {a0}, s);
  return o;
}
static Tensor transpose(const Tensor& a);
struct TransposeNode : Node {
  TransposeNode() { name = "transpose"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {transpose(g)}; }
};
static Tensor transpose(const Tensor& a) {          // a view: no copy
  if (a->shape.size() != 2) { g_last_error = "transpose expects a matrix"; return nullptr; }
  auto t = std::make_shared<TensorImpl>();
  t->storage = a->storage;
  t->offset = a->offset;
  t->shape = {a->shape[1], a->shape[0]};
  t->strides = {a->strides[1], a->strides[0]};
  attach<TransposeNode>(t, {a});
  return t;
}
// C[M,N] = A[M,K] B[K,N], blocked over k for cache reuse
static void gemm_raw(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K) {
  std::fill(C, C + M * N, 0.f);
  constexpr int64_t KB = 64;
  for (int64_t k0 = 0; k0 < K; k0 += KB) {
    const int64_t k1 = std::min(K, k0 + KB);
    for (int64_t i = 0; i < M; i++) {
      float* c = C + i * N;
      for (int64_t k = k0; k < k1; k++) {
        const float a = A[i * K + k];
        const float* b = B + k * N;
        for (int64_t j = 0; j < N; j++) c[j] += a * b[j];
      }
    }
  }
}
static Tensor matmul(const Tensor& a0, const Tensor& b0);
struct MatmulNode : Node {
  Tensor a, b;
  MatmulNode(Tensor x, Tensor y) : a(std::move(x)), b(std::move(y)) { name = "matmul"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    const bool prev = g_grad_enabled;
    g_grad_enabled = false;
    Tensor ga = inputs[0] ? matmul(g, transpose(b)) : nullptr, gb = inputs[1] ? matmul(transpose(a), g) : nullptr;
    g_grad_enabled = prev;
    return {ga, gb};
  }
};
static Tensor matmul(const Tensor& a0, const Tensor& b0) {
  if (a0->shape.size() != 2 || b0->shape.size() != 2 || a0->shape[1] != b0->shape[0]) { g_last_error = "matmul: shapes do not match"; return nullptr; }
  Tensor a = contiguous(a0), b = contiguous(b0);
  Tensor o = make({a->shape[0], b->shape[1]});
  gemm_raw(a->data(), b->data(), o->data(), a->shape[0], b->shape[1], a->shape[1]);
  attach<MatmulNode>(o, {a0, b0}, a, b);
  return o;
}
enum class Act { Relu, Tanh, Sigmoid };
struct ActNode : Node {
  Act k; Tensor y, x;
  ActNode(Act kk, Tensor out, Tensor in) : k(kk), y(std::move(out)), x(std::move(in)) { name = "activation"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(gc->shape);
    for (int64_t i = 0; i < gc->numel(); i++) {
      const float v = y->data()[i];
      const float d = k == Act::Relu ? (x->data()[i] > 0.f ? 1.f : 0.f) : (k == Act::Tanh ? 1.f - v * v : v * (1.f - v));
      o->data()[i] = gc->data()[i] * d;
    }
    return {o};
  }
};
static Tensor activation(Act k, const Tensor& a0) {
  Tensor a = contiguous(a0), o = make(a->shape);
  for (int64_t i = 0; i < a->numel(); i++) {
    const float x = a->data()[i];
    o->data()[i] = k == Act::Relu ? (x > 0.f ? x : 0.f) : (k == Act::Tanh ? std::tanh(x) : 1.f / (1.f + std::exp(-x)));
  }
  attach<ActNode>(o, {a0}, k, o, a);
  return o;
}
struct SumNode : Node {
  std::vector<int64_t> shape; float w;
  SumNode(std::vector<int64_t> s, float ww) : shape(std::move(s)), w(ww) { name = "sum"; }
  std::vector<Tensor> backward(const Tensor& g) override { return {make(shape, g->data()[0] * w)}; }
};
static Tensor sum(const Tensor& a0, bool mean) {
  Tensor a = contiguous(a0), o = make({});
  double s = 0;
  for (int64_t i = 0; i < a->numel(); i++) s += a->data()[i];
  const float w = mean ? 1.f / (float)std::max<int64_t>(a->numel(), 1) : 1.f;
  o->data()[0] = (float)(s * w);
  attach<SumNode>(o, {a0}, a->shape, w);
  return o;
}
// mean over rows of -log softmax(logits)[target]
struct CrossEntropyNode : Node {
  Tensor prob; std::vector<int64_t> tgt;
  CrossEntropyNode(Tensor p, std::vector<int64_t> t) : prob(std::move(p)), tgt(std::move(t)) { name = "cross_entropy"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    const int64_t R = prob->shape[0], C = prob->shape[1];
    Tensor o = make(prob->shape);
    const float s = g->data()[0] / (float)R;
    for (int64_t r = 0; r < R; r++)
      for (int64_t c = 0; c < C; c++) o->data()[r * C + c] = (prob->data()[r * C + c] - (c == tgt[r] ? 1.f : 0.f)) * s;
    return {o};
  }
};
static Tensor cross_entropy(const Tensor& l0, const int64_t* targets, int64_t n) {
  if (l0->shape.size() != 2 || l0->shape[0] != n) { g_last_error = "cross_entropy: logits [rows, classes] and one target per row"; return nullptr; }
  Tensor l = contiguous(l0), prob = make(l->shape), o = make({});
  const int64_t R = l->shape[0], C = l->shape[1];
  double total = 0;
  for (int64_t r = 0; r < R; r++) {
    if (targets[r] < 0 || targets[r] >= C) { g_last_error = "cross_entropy: target out of range"; return nullptr; }
    const float* x = l->data() + r * C;
    float m = x[0];
    for (int64_t c = 1; c < C; c++) m = std::max(m, x[c]);
    double z = 0;
    for (int64_t c = 0; c < C; c++) z += std::exp((double)x[c] - m);
    const double lz = std::log(z) + m;
    for (int64_t c = 0; c < C; c++) prob->data()[r * C + c] = (float)std::exp((double)x[c] - lz);
    total += lz - x[targets[r]];
  }
  o->data()[0] = (float)(total / (double)R);
  attach<CrossEntropyNode>(o, {l0}, prob, std::vector<int64_t>(targets, targets + n));
  return o;
}
static Tensor linear(const Tensor& x, const Tensor& w, const Tensor& b) {     // x W^T + b with W [out, in]
  Tensor y = matmul(x, transpose(w));
  if (!y) return nullptr;
  return b ? binary(Bin::Add, y, b) : y;
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// SGD
// ---------------------------------------------------------------------------------------------------------------------------------------
struct Sgd {
  std::vector<Tensor> params;
  std::vector<std::vector<float>> buf;
  float lr, momentum, dampening, weight_decay;
  bool nesterov;
  bool first = true;
  void step() {
    if (buf.size() != params.size()) buf.resize(params.size());
    for (size_t k = 0; k < params.size(); k++) {
      Tensor& p = params[k];
      if (!p->grad) continue;
      Tensor gc = contiguous(p->grad);
      const int64_t n = p->numel();
      float* w = p->data();
      if (!p->is_contiguous()) continue;            // parameters are created contiguous; views are not optimised
      std::vector<float>& m = buf[k];
      const bool init = m.empty();
      if (momentum != 0.f && init) m.assign((size_t)n, 0.f);
      for (int64_t i = 0; i < n; i++) {
        float g = gc->data()[i] + weight_decay * w[i];
        if (momentum != 0.f) {
          m[i] = init ? g : momentum * m[i] + (1.f - dampening) * g;
          g = nesterov ? g + momentum * m[i] : m[i];
        }
        w[i] -= lr * g;
      }
      p->version++;
    }
  }
};

// ---------------------------------------------------------------------------------------------------------------------------------------
// more operations: element-wise family, division, reshape, reductions along one dimension, softmax, convolution, pooling
// ---------------------------------------------------------------------------------------------------------------------------------------
enum class Un { Exp = 0, Log = 1, Sqrt = 2, Gelu = 3, Silu = 4, LeakyRelu = 5, Pow = 6, Abs = 7, Square = 8, Reciprocal = 9 };
static inline float un_fwd(Un k, float x, float p) {
  switch (k) {
    case Un::Exp: return std::exp(x);
    case Un::Log: return std::log(x);
    case Un::Sqrt: return std::sqrt(x);
    case Un::Gelu: return 0.5f * x * (1.f + std::erf(x * 0.70710678118654752f));
    case Un::Silu: return x / (1.f + std::exp(-x));
    case Un::LeakyRelu: return x > 0.f ? x : p * x;
    case Un::Pow: return std::pow(x, p);
    case Un::Abs: return std::fabs(x);
    case Un::Square: return x * x;
    case Un::Reciprocal: return 1.f / x;
  }
  return 0.f;
}
static inline float un_bwd(Un k, float x, float y, float p) {      // d out / d in from the input x and the output y
  switch (k) {
    case Un::Exp: return y;
    case Un::Log: return 1.f / x;
    case Un::Sqrt: return 0.5f / y;
    case Un::Gelu: return 0.5f * (1.f + std::erf(x * 0.70710678118654752f)) + x * 0.3989422804014327f * std::exp(-0.5f * x * x);
    case Un::Silu: { const float sg = 1.f / (1.f + std::exp(-x)); return sg * (1.f + x * (1.f - sg)); }
    case Un::LeakyRelu: return x > 0.f ? 1.f : p;
    case Un::Pow: return p * std::pow(x, p - 1.f);
    case Un::Abs: return x > 0.f ? 1.f : (x < 0.f ? -1.f : 0.f);
    case Un::Square: return 2.f * x;
    case Un::Reciprocal: return -y * y;
  }
  return 0.f;
}
struct UnaryNode : Node {
  Un k; float p; Tensor x, y;
  UnaryNode(Un kk, float pp, Tensor in, Tensor out) : k(kk), p(pp), x(std::move(in)), y(std::move(out)) { name = "unary"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(gc->shape);
    for (int64_t i = 0; i < gc->numel(); i++) o->data()[i] = gc->data()[i] * un_bwd(k, x->data()[i], y->data()[i], p);
    return {o};
  }
};
static Tensor unary(Un k, const Tensor& a0, float p) {
  Tensor a = contiguous(a0), o = make(a->shape);
  for (int64_t i = 0; i < a->numel(); i++) o->data()[i] = un_fwd(k, a->data()[i], p);
  attach<UnaryNode>(o, {a0}, k, p, a, o);
  return o;
}

// a / b with the row-broadcast rule of the other binary operations
struct DivNode : Node {
  Tensor a, b;
  DivNode(Tensor x, Tensor y) : a(std::move(x)), b(std::move(y)) { name = "div"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), ga = make(a->shape), gb = make(a->shape);
    const int64_t n = gc->numel(), nb = b->numel();
    for (int64_t i = 0; i < n; i++) {
      const float d = b->data()[i % nb];
      ga->data()[i] = gc->data()[i] / d;
      gb->data()[i] = -gc->data()[i] * a->data()[i] / (d * d);
    }
    return {ga, reduce_to(gb, b->shape)};
  }
};
static Tensor divide(const Tensor& a0, const Tensor& b0) {
  Tensor a = contiguous(a0), b = contiguous(b0);
  const int64_t n = a->numel(), nb = b->numel();
  if (!suffix_broadcast_ok(a->shape, b->shape)) { g_last_error = "div: shapes do not match or broadcast"; return nullptr; }
  Tensor o = make(a->shape);
  for (int64_t i = 0; i < n; i++) o->data()[i] = a->data()[i] / b->data()[i % nb];
  attach<DivNode>(o, {a0, b0}, a, b);
  return o;
}

static Tensor reshape(const Tensor& a0, const std::vector<int64_t>& shape);
struct ReshapeNode : Node {
  std::vector<int64_t> from;
  explicit ReshapeNode(std::vector<int64_t> s) : from(std::move(s)) { name = "reshape"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    const bool prev = g_grad_enabled;
    g_grad_enabled = false;
    Tensor o = reshape(g, from);
    g_grad_enabled = prev;
    return {o};
  }
};
static Tensor reshape(const Tensor& a0, const std::vector<int64_t>& shape_in) {       // a view of the (contiguous copy of the) storage; one -1 is inferred
  std::vector<int64_t> shape = shape_in;
  int64_t known = 1, infer = -1;
  for (size_t i = 0; i < shape.size(); i++) {
    if (shape[i] == -1) { if (infer >= 0) { g_last_error = "reshape: only one dimension can be inferred"; return nullptr; } infer = (int64_t)i; }
    else if (shape[i] < 0) { g_last_error = "reshape: negative dimension"; return nullptr; }
    else known *= shape[i];
  }
  if (infer >= 0) { if (known == 0 || a0->numel() % known) { g_last_error = "reshape: cannot infer the dimension"; return nullptr; } shape[(size_t)infer] = a0->numel() / known; known *= shape[(size_t)infer]; }
  if (known != a0->numel()) { g_last_error = "reshape: element counts differ"; return nullptr; }
  Tensor a = contiguous(a0);
  auto t = std::make_shared<TensorImpl>();
  t->storage = a->storage;
  t->offset = a->offset;
  t->shape = shape;
  t->strides = row_major(shape);
  attach<ReshapeNode>(t, {a0}, a0->shape);
  return t;
}

// sum (or mean) along one dimension: the tensor is seen as [outer, len, inner]
struct SumDimNode : Node {
  std::vector<int64_t> shape; int64_t outer, len, inner; float w;
  SumDimNode(std::vector<int64_t> s, int64_t o, int64_t l, int64_t i, float ww) : shape(std::move(s)), outer(o), len(l), inner(i), w(ww) { name = "sum_dim"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(shape);
    for (int64_t a = 0; a < outer; a++)
      for (int64_t l = 0; l < len; l++)
        for (int64_t i = 0; i < inner; i++) o->data()[(a * len + l) * inner + i] = gc->data()[a * inner + i] * w;
    return {o};
  }
};
static Tensor sum_dim(const Tensor& a0, int dim, bool keepdim, bool mean) {
  const int nd = (int)a0->shape.size();
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd) { g_last_error = "sum: dimension out of range"; return nullptr; }
  Tensor a = contiguous(a0);
  int64_t outer = 1, inner = 1;
  const int64_t len = a->shape[(size_t)dim];
  for (int i = 0; i < dim; i++) outer *= a->shape[(size_t)i];
  for (int i = dim + 1; i < nd; i++) inner *= a->shape[(size_t)i];
  std::vector<int64_t> os;
  for (int i = 0; i < nd; i++) { if (i != dim) os.push_back(a->shape[(size_t)i]); else if (keepdim) os.push_back(1); }
  Tensor o = make(os);
  const float w = mean ? 1.f / (float)std::max<int64_t>(len, 1) : 1.f;
  for (int64_t x = 0; x < outer; x++)
    for (int64_t i = 0; i < inner; i++) {
      double s = 0;
      for (int64_t l = 0; l < len; l++) s += a->data()[(x * len + l) * inner + i];
      o->data()[x * inner + i] = (float)(s * w);
    }
  attach<SumDimNode>(o, {a0}, a->shape, outer, len, inner, w);
  return o;
}

// softmax / log-softmax over the last dimension
struct SoftmaxNode : Node {
  Tensor y; bool log;
  SoftmaxNode(Tensor out, bool l) : y(std::move(out)), log(l) { name = "softmax"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(gc->shape);
    const int64_t C = y->shape.back(), R = y->numel() / std::max<int64_t>(C, 1);
    for (int64_t r = 0; r < R; r++) {
      const float* yy = y->data() + r * C;
      const float* gg = gc->data() + r * C;
      double dot = 0;
      for (int64_t c = 0; c < C; c++) dot += log ? gg[c] : gg[c] * yy[c];
      for (int64_t c = 0; c < C; c++) o->data()[r * C + c] = log ? gg[c] - std::exp(yy[c]) * (float)dot : yy[c] * (gg[c] - (float)dot);
    }
    return {o};
  }
};
static Tensor softmax(const Tensor& a0, bool log) {
  if (a0->shape.empty()) { g_last_error = "softmax needs at least one dimension"; return nullptr; }
  Tensor a = contiguous(a0), o = make(a->shape);
  const int64_t C = a->shape.back(), R = a->numel() / std::max<int64_t>(C, 1);
  for (int64_t r = 0; r < R; r++) {
    const float* x = a->data() + r * C;
    float m = x[0];
    for (int64_t c = 1; c < C; c++) m = std::max(m, x[c]);
    double z = 0;
    for (int64_t c = 0; c < C; c++) z += std::exp((double)x[c] - m);
    const double lz = std::log(z) + m;
    for (int64_t c = 0; c < C; c++) o->data()[r * C + c] = log ? (float)(x[c] - lz) : (float)std::exp((double)x[c] - lz);
  }
  attach<SoftmaxNode>(o, {a0}, o, log);
  return o;
}

// 2-d convolution (NCHW, weight [O, C, kh, kw]) as patch matrix x GEMM, image by image
struct ConvGeom { int64_t N, C, H, W, O, kh, kw, sh, sw, ph, pw, Ho, Wo; };
static void im2col(const float* x, const ConvGeom& g, float* col) {          // col [C*kh*kw, Ho*Wo]
  for (int64_t c = 0; c < g.C; c++)
    for (int64_t i = 0; i < g.kh; i++)
      for (int64_t j = 0; j < g.kw; j++) {
        float* row = col + ((c * g.kh + i) * g.kw + j) * g.Ho * g.Wo;
        for (int64_t oy = 0; oy < g.Ho; oy++) {
          const int64_t iy = oy * g.sh - g.ph + i;
          for (int64_t ox = 0; ox < g.Wo; ox++) {
            const int64_t ix = ox * g.sw - g.pw + j;
            row[oy * g.Wo + ox] = (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) ? x[(c * g.H + iy) * g.W + ix] : 0.f;
          }
        }
      }
}
static void col2im_add(const float* col, const ConvGeom& g, float* x) {
  for (int64_t c = 0; c < g.C; c++)
    for (int64_t i = 0; i < g.kh; i++)
      for (int64_t j = 0; j < g.kw; j++) {
        const float* row = col + ((c * g.kh + i) * g.kw + j) * g.Ho * g.Wo;
        for (int64_t oy = 0; oy < g.Ho; oy++) {
          const int64_t iy = oy * g.sh - g.ph + i;
          if (iy < 0 || iy >= g.H) continue;
          for (int64_t ox = 0; ox < g.Wo; ox++) {
            const int64_t ix = ox * g.sw - g.pw + j;
            if (ix >= 0 && ix < g.W) x[(c * g.H + iy) * g.W + ix] += row[oy * g.Wo + ox];
          }
        }
      }
}
struct Conv2dNode : Node {
  Tensor x, w; ConvGeom g; bool has_bias;
  Conv2dNode(Tensor xx, Tensor ww, ConvGeom gg, bool hb) : x(std::move(xx)), w(std::move(ww)), g(gg), has_bias(hb) { name = "conv2d"; }
  std::vector<Tensor> backward(const Tensor& gout) override {
    Tensor gy = contiguous(gout);
    const int64_t K = g.C * g.kh * g.kw, P = g.Ho * g.Wo;
    Tensor gx = inputs[0] ? make(x->shape) : nullptr, gw = inputs[1] ? make(w->shape) : nullptr, gb = (has_bias && inputs[2]) ? make({g.O}) : nullptr;
    std::vector<float> col((size_t)(K * P)), tmp((size_t)std::max(K * P, g.O * K)), wt((size_t)(K * g.O));
    for (int64_t o = 0; o < g.O; o++)
      for (int64_t k = 0; k < K; k++) wt[(size_t)(k * g.O + o)] = w->data()[o * K + k];
    for (int64_t n = 0; n < g.N; n++) {
      const float* gyn = gy->data() + n * g.O * P;
      if (gw) {                                          // dW += dY [O, P] x col^T [P, K]
        im2col(x->data() + n * g.C * g.H * g.W, g, col.data());
        for (int64_t o = 0; o < g.O; o++)
          for (int64_t k = 0; k < K; k++) {
            const float* a = gyn + o * P;
            const float* b = col.data() + k * P;
            float sacc = 0.f;
            for (int64_t q = 0; q < P; q++) sacc += a[q] * b[q];
            gw->data()[o * K + k] += sacc;
          }
      }
      if (gx) {                                          // dcol [K, P] = W^T [K, O] x dY [O, P], scattered back
        gemm_raw(wt.data(), gyn, tmp.data(), K, P, g.O);
        col2im_add(tmp.data(), g, gx->data() + n * g.C * g.H * g.W);
      }
      if (gb)
        for (int64_t o = 0; o < g.O; o++) {
          float sacc = 0.f;
          for (int64_t q = 0; q < P; q++) sacc += gyn[o * P + q];
          gb->data()[o] += sacc;
        }
    }
    std::vector<Tensor> out{gx, gw};
    if (has_bias) out.push_back(gb);
    return out;
  }
};
static Tensor conv2d(const Tensor& x0, const Tensor& w0, const Tensor& b0, int sh, int sw, int ph, int pw) {
  if (x0->shape.size() != 4 || w0->shape.size() != 4 || x0->shape[1] != w0->shape[1] || sh < 1 || sw < 1 || ph < 0 || pw < 0 ||
      (b0 && (b0->shape.size() != 1 || b0->shape[0] != w0->shape[0]))) { g_last_error = "conv2d: x [N, C, H, W], weight [O, C, kh, kw], bias [O], stride >= 1, padding >= 0"; return nullptr; }
  Tensor x = contiguous(x0), w = contiguous(w0), b = b0 ? contiguous(b0) : nullptr;
  ConvGeom g{x->shape[0], x->shape[1], x->shape[2], x->shape[3], w->shape[0], w->shape[2], w->shape[3], sh, sw, ph, pw, 0, 0};
  g.Ho = (g.H + 2 * g.ph - g.kh) / g.sh + 1;
  g.Wo = (g.W + 2 * g.pw - g.kw) / g.sw + 1;
  if (g.H + 2 * g.ph < g.kh || g.W + 2 * g.pw < g.kw) { g_last_error = "conv2d: kernel larger than the padded input"; return nullptr; }
  const int64_t K = g.C * g.kh * g.kw, P = g.Ho * g.Wo;
  Tensor o = make({g.N, g.O, g.Ho, g.Wo});
  std::vector<float> col((size_t)(K * P));
  for (int64_t n = 0; n < g.N; n++) {
    im2col(x->data() + n * g.C * g.H * g.W, g, col.data());
    float* on = o->data() + n * g.O * P;
    gemm_raw(w->data(), col.data(), on, g.O, P, K);
    if (b)
      for (int64_t oc = 0; oc < g.O; oc++)
        for (int64_t q = 0; q < P; q++) on[oc * P + q] += b->data()[oc];
  }
  if (b0) attach<Conv2dNode>(o, {x0, w0, b0}, x, w, g, true);
  else attach<Conv2dNode>(o, {x0, w0}, x, w, g, false);
  return o;
}

// max pooling over k x k windows with the given stride (no padding); the position of each maximum is kept for the backward pass
struct MaxPoolNode : Node {
  std::vector<int64_t> shape; std::vector<int64_t> arg;
  MaxPoolNode(std::vector<int64_t> s, std::vector<int64_t> a) : shape(std::move(s)), arg(std::move(a)) { name = "max_pool2d"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(shape);
    for (int64_t i = 0; i < gc->numel(); i++) o->data()[arg[(size_t)i]] += gc->data()[i];
    return {o};
  }
};
static Tensor max_pool2d(const Tensor& x0, int k, int stride) {
  if (x0->shape.size() != 4 || k < 1 || stride < 1 || x0->shape[2] < k || x0->shape[3] < k) { g_last_error = "max_pool2d: x [N, C, H, W] with H, W >= kernel"; return nullptr; }
  Tensor x = contiguous(x0);
  const int64_t N = x->shape[0], C = x->shape[1], Hh = x->shape[2], Ww = x->shape[3], Ho = (Hh - k) / stride + 1, Wo = (Ww - k) / stride + 1;
  Tensor o = make({N, C, Ho, Wo});
  std::vector<int64_t> arg((size_t)o->numel());
  for (int64_t nc = 0; nc < N * C; nc++)
    for (int64_t oy = 0; oy < Ho; oy++)
      for (int64_t ox = 0; ox < Wo; ox++) {
        int64_t best = (nc * Hh + oy * stride) * Ww + ox * stride;
        for (int64_t i = 0; i < k; i++)
          for (int64_t j = 0; j < k; j++) {
            const int64_t at = (nc * Hh + oy * stride + i) * Ww + ox * stride + j;
            if (x->data()[at] > x->data()[best]) best = at;
          }
        const int64_t oi = (nc * Ho + oy) * Wo + ox;
        o->data()[oi] = x->data()[best];
        arg[(size_t)oi] = best;
      }
  attach<MaxPoolNode>(o, {x0}, x->shape, std::move(arg));
  return o;
}



// a view of `len` consecutive entries of dimension `dim` starting at `start`
struct NarrowNode : Node {
  std::vector<int64_t> shape; int dim; int64_t start;
  NarrowNode(std::vector<int64_t> s, int d, int64_t st) : shape(std::move(s)), dim(d), start(st) { name = "narrow"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(shape);
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < dim; i++) outer *= shape[(size_t)i];
    for (size_t i = (size_t)dim + 1; i < shape.size(); i++) inner *= shape[i];
    const int64_t full = shape[(size_t)dim], len = gc->shape[(size_t)dim];
    for (int64_t a = 0; a < outer; a++)
      std::memcpy(o->data() + (a * full + start) * inner, gc->data() + a * len * inner, sizeof(float) * (size_t)(len * inner));
    return {o};
  }
};
static Tensor narrow(const Tensor& a, int dim, int64_t start, int64_t len) {
  const int nd = (int)a->shape.size();
  if (dim < 0) dim += nd;
  if (dim < 0 || dim >= nd || start < 0 || len < 0 || start + len > a->shape[(size_t)dim]) { g_last_error = "narrow: range outside the dimension"; return nullptr; }
  auto t = std::make_shared<TensorImpl>();
  t->storage = a->storage;
  t->offset = a->offset + start * a->strides[(size_t)dim];
  t->shape = a->shape;
  t->shape[(size_t)dim] = len;
  t->strides = a->strides;
  attach<NarrowNode>(t, {a}, a->shape, dim, start);
  return t;
}

// a view with permuted dimensions
static Tensor permute(const Tensor& a, const std::vector<int64_t>& dims);
struct PermuteNode : Node {
  std::vector<int64_t> inverse;
  explicit PermuteNode(std::vector<int64_t> inv) : inverse(std::move(inv)) { name = "permute"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    const bool prev = g_grad_enabled;
    g_grad_enabled = false;
    Tensor o = permute(g, inverse);
    g_grad_enabled = prev;
    return {o};
  }
};
static Tensor permute(const Tensor& a, const std::vector<int64_t>& dims) {
  const size_t nd = a->shape.size();
  std::vector<int64_t> inv(nd, -1);
  if (dims.size() != nd) { g_last_error = "permute: one entry per dimension"; return nullptr; }
  for (size_t i = 0; i < nd; i++) {
    const int64_t d = dims[i] < 0 ? dims[i] + (int64_t)nd : dims[i];
    if (d < 0 || d >= (int64_t)nd || inv[(size_t)d] >= 0) { g_last_error = "permute: not a permutation"; return nullptr; }
    inv[(size_t)d] = (int64_t)i;
  }
  auto t = std::make_shared<TensorImpl>();
  t->storage = a->storage;
  t->offset = a->offset;
  for (size_t i = 0; i < nd; i++) {
    const int64_t d = dims[i] < 0 ? dims[i] + (int64_t)nd : dims[i];
    t->shape.push_back(a->shape[(size_t)d]);
    t->strides.push_back(a->strides[(size_t)d]);
  }
  attach<PermuteNode>(t, {a}, inv);
  return t;
}

// batched matrix product: [..., M, K] x [..., K, N] with equal leading dimensions
struct BmmNode : Node {
  Tensor a, b;
  BmmNode(Tensor x, Tensor y) : a(std::move(x)), b(std::move(y)) { name = "bmm"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g);
    const size_t nd = a->shape.size();
    const int64_t M = a->shape[nd - 2], K = a->shape[nd - 1], N = b->shape[nd - 1], B = a->numel() / std::max<int64_t>(M * K, 1);
    Tensor ga = inputs[0] ? make(a->shape) : nullptr, gb = inputs[1] ? make(b->shape) : nullptr;
    std::vector<float> bt((size_t)(N * K)), at((size_t)(K * M));
    for (int64_t i = 0; i < B; i++) {
      const float* A = a->data() + i * M * K;
      const float* Bm = b->data() + i * K * N;
      const float* G = gc->data() + i * M * N;
      if (ga) {                                          // dA = G [M, N] x B^T [N, K]
        for (int64_t k = 0; k < K; k++)
          for (int64_t n = 0; n < N; n++) bt[(size_t)(n * K + k)] = Bm[k * N + n];
        gemm_raw(G, bt.data(), ga->data() + i * M * K, M, K, N);
      }
      if (gb) {                                          // dB = A^T [K, M] x G [M, N]
        for (int64_t m = 0; m < M; m++)
          for (int64_t k = 0; k < K; k++) at[(size_t)(k * M + m)] = A[m * K + k];
        gemm_raw(at.data(), G, gb->data() + i * K * N, K, N, M);
      }
    }
    return {ga, gb};
  }
};
static Tensor bmm(const Tensor& a0, const Tensor& b0) {
  const size_t nd = a0->shape.size();
  if (nd < 2 || b0->shape.size() != nd || a0->shape[nd - 1] != b0->shape[nd - 2]) { g_last_error = "bmm: [..., M, K] x [..., K, N] with equal leading dimensions"; return nullptr; }
  for (size_t i = 0; i + 2 < nd; i++)
    if (a0->shape[i] != b0->shape[i]) { g_last_error = "bmm: leading dimensions differ"; return nullptr; }
  Tensor a = contiguous(a0), b = contiguous(b0);
  const int64_t M = a->shape[nd - 2], K = a->shape[nd - 1], N = b->shape[nd - 1], B = a->numel() / std::max<int64_t>(M * K, 1);
  std::vector<int64_t> os(a->shape.begin(), a->shape.end() - 1);
  os.push_back(N);
  Tensor o = make(os);
  for (int64_t i = 0; i < B; i++) gemm_raw(a->data() + i * M * K, b->data() + i * K * N, o->data() + i * M * N, M, N, K);
  attach<BmmNode>(o, {a0, b0}, a, b);
  return o;
}

// layer normalisation over the last dimension with an optional scale and shift
struct LayerNormNode : Node {
  Tensor xhat, w; std::vector<float> rstd; bool has_w, has_b;
  LayerNormNode(Tensor xh, Tensor ww, std::vector<float> r, bool hw, bool hb) : xhat(std::move(xh)), w(std::move(ww)), rstd(std::move(r)), has_w(hw), has_b(hb) { name = "layer_norm"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g);
    const int64_t C = xhat->shape.back(), R = xhat->numel() / std::max<int64_t>(C, 1);
    Tensor gx = inputs[0] ? make(xhat->shape) : nullptr;
    Tensor gw = (has_w && inputs[1]) ? make({C}) : nullptr;
    Tensor gb = (has_b && inputs[has_w ? 2 : 1]) ? make({C}) : nullptr;
    for (int64_t r = 0; r < R; r++) {
      const float* gg = gc->data() + r * C;
      const float* xh = xhat->data() + r * C;
      double s1 = 0, s2 = 0;
      for (int64_t c = 0; c < C; c++) {
        const float gy = has_w ? gg[c] * w->data()[c] : gg[c];
        s1 += gy;
        s2 += gy * xh[c];
        if (gw) gw->data()[c] += gg[c] * xh[c];
        if (gb) gb->data()[c] += gg[c];
      }
      if (gx)
        for (int64_t c = 0; c < C; c++) {
          const float gy = has_w ? gg[c] * w->data()[c] : gg[c];
          gx->data()[r * C + c] = rstd[(size_t)r] * (gy - (float)(s1 / C) - xh[c] * (float)(s2 / C));
        }
    }
    std::vector<Tensor> out{gx};
    if (has_w) out.push_back(gw);
    if (has_b) out.push_back(gb);
    return out;
  }
};
static Tensor layer_norm(const Tensor& x0, const Tensor& w0, const Tensor& b0, float eps) {
  if (x0->shape.empty()) { g_last_error = "layer_norm needs at least one dimension"; return nullptr; }
  const int64_t C = x0->shape.back();
  if ((w0 && (w0->shape.size() != 1 || w0->shape[0] != C)) || (b0 && (b0->shape.size() != 1 || b0->shape[0] != C))) { g_last_error = "layer_norm: scale and shift have the length of the last dimension"; return nullptr; }
  Tensor x = contiguous(x0), w = w0 ? contiguous(w0) : nullptr, b = b0 ? contiguous(b0) : nullptr, o = make(x->shape), xh = make(x->shape);
  const int64_t R = x->numel() / std::max<int64_t>(C, 1);
  std::vector<float> rstd((size_t)R);
  for (int64_t r = 0; r < R; r++) {
    const float* xx = x->data() + r * C;
    double m = 0, v = 0;
    for (int64_t c = 0; c < C; c++) m += xx[c];
    m /= (double)C;
    for (int64_t c = 0; c < C; c++) v += (xx[c] - m) * (xx[c] - m);
    const float rs = (float)(1.0 / std::sqrt(v / (double)C + eps));
    rstd[(size_t)r] = rs;
    for (int64_t c = 0; c < C; c++) {
      const float h = (float)(xx[c] - m) * rs;
      xh->data()[r * C + c] = h;
      o->data()[r * C + c] = (w ? h * w->data()[c] : h) + (b ? b->data()[c] : 0.f);
    }
  }
  if (w0 && b0) attach<LayerNormNode>(o, {x0, w0, b0}, xh, w, rstd, true, true);
  else if (w0) attach<LayerNormNode>(o, {x0, w0}, xh, w, rstd, true, false);
  else if (b0) attach<LayerNormNode>(o, {x0, b0}, xh, w, rstd, false, true);
  else attach<LayerNormNode>(o, {x0}, xh, w, rstd, false, false);
  return o;
}

// rows of a table selected by integer ids: out [..., D] for ids [...]
struct EmbeddingNode : Node {
  std::vector<int64_t> ids, table_shape;
  EmbeddingNode(std::vector<int64_t> i, std::vector<int64_t> ts) : ids(std::move(i)), table_shape(std::move(ts)) { name = "embedding"; }
  std::vector<Tensor> backward(const Tensor& g) override {
    Tensor gc = contiguous(g), o = make(table_shape);
    const int64_t D = table_shape[1];
    for (size_t r = 0; r < ids.size(); r++)
      for (int64_t d = 0; d < D; d++) o->data()[ids[r] * D + d] += gc->data()[(int64_t)r * D + d];
    return {o};
  }
};
static Tensor embedding(const Tensor& table0, const int64_t* ids, const int64_t* ids_shape, int ids_ndim) {
  if (table0->shape.size() != 2) { g_last_error = "embedding: the table is [rows, dim]"; return nullptr; }
  Tensor table = contiguous(table0);
  const int64_t V = table->shape[0], D = table->shape[1];
  std::vector<int64_t> os(ids_shape, ids_shape + ids_ndim);
  int64_t n = 1;
  for (auto v : os) n *= v;
  os.push_back(D);
  Tensor o = make(os);
  for (int64_t r = 0; r < n; r++) {
    if (ids[r] < 0 || ids[r] >= V) { g_last_error = "embedding: id out of range"; return nullptr; }
    std::memcpy(o->data() + r * D, table->data() + ids[r] * D, sizeof(float) * (size_t)D);
  }
  attach<EmbeddingNode>(o, {table0}, std::vector<int64_t>(ids, ids + n), table->shape);
  return o;
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// Adam / AdamW (decoupled decay when `decoupled`, else the decay is added to the gradient), bias-corrected, same rule as the device kernel
// ---------------------------------------------------------------------------------------------------------------------------------------
struct Adam {
  std::vector<Tensor> params;
  std::vector<std::vector<float>> m, v;
  float lr, beta1, beta2, eps, weight_decay;
  bool decoupled;
  int64_t t = 0;
  void step() {
    if (m.size() != params.size()) { m.resize(params.size()); v.resize(params.size()); }
    t++;
    const double c1 = 1.0 - std::pow((double)beta1, (double)t), c2 = 1.0 - std::pow((double)beta2, (double)t);
    for (size_t k = 0; k < params.size(); k++) {
      Tensor& p = params[k];
      if (!p->grad || !p->is_contiguous()) continue;
      Tensor gc = contiguous(p->grad);
      const int64_t n = p->numel();
      if (m[k].empty()) { m[k].assign((size_t)n, 0.f); v[k].assign((size_t)n, 0.f); }
      float* w = p->data();
      for (int64_t i = 0; i < n; i++) {
        float g = gc->data()[i];
        if (decoupled) w[i] *= 1.f - lr * weight_decay;
        else g += weight_decay * w[i];
        m[k][(size_t)i] = beta1 * m[k][(size_t)i] + (1.f - beta1) * g;
        v[k][(size_t)i] = beta2 * v[k][(size_t)i] + (1.f - beta2) * g * g;
        const double mh = m[k][(size_t)i] / c1, vh = v[k][(size_t)i] / c2;
        w[i] -= (float)(lr * mh / (std::sqrt(vh) + eps));
      }
      p->version++;
    }
  }
};

}  // namespace ft

// ---------------------------------------------------------------------------------------------------------------------------------------
// C ABI: a handle is a heap-allocated ft::Tensor (shared_ptr); every function that returns a handle returns null on error
// (ftc_last_error gives the reason). Handles are released with ftc_free.
// ---------------------------------------------------------------------------------------------------------------------------------------
using ft::Tensor;
static Tensor* H(const Tensor& t) { return t ? new Tensor(t) : nullptr; }
static const Tensor& T(const void* h) { return *static_cast<const Tensor*>(h); }

// Last error message of the calling thread ("" if none).
FT_API const char* ftc_last_error() { return ft::g_last_error.c_str(); }
// New tensor of the given shape; data (may be null: zeros) is copied. requires_grad marks it as a leaf that accumulates .grad.
FT_API void* ftc_tensor_new(const float* data, const int64_t* shape, int ndim, int requires_grad) {
  Tensor t = ft::make(std::vector<int64_t>(shape, shape + ndim));
  if (data) std::memcpy(t->data(), data, sizeof(float) * (size_t)t->numel());
  t->requires_grad = requires_grad != 0;
  return H(t);
}
FT_API void ftc_free(void* h) { delete static_cast<Tensor*>(h); }
FT_API int ftc_ndim(const void* h) { return (int)T(h)->shape.size(); }
FT_API int64_t ftc_numel(const void* h) { return T(h)->numel(); }
FT_API void ftc_shape(const void* h, int64_t* out) { for (size_t i = 0; i < T(h)->shape.size(); i++) out[i] = T(h)->shape[i]; }
FT_API uint64_t ftc_id(const void* h) { return T(h)->id; }
FT_API int ftc_requires_grad(const void* h) { return T(h)->requires_grad ? 1 : 0; }
FT_API int ftc_is_leaf(const void* h) { return T(h)->is_leaf() ? 1 : 0; }
FT_API const char* ftc_grad_fn_name(const void* h) { return T(h)->grad_fn ? T(h)->grad_fn->name : ""; }
// Pointer to the tensor's own storage when it is contiguous (shared with the caller: writes are visible to the tensor), else null.
FT_API float* ftc_data_ptr(void* h) { return T(h)->is_contiguous() ? const_cast<float*>(T(h)->data()) : nullptr; }
// Copies the values out in row-major order.
FT_API void ftc_copy_out(const void* h, float* out) { Tensor c = ft::contiguous(T(h)); std::memcpy(out, c->data(), sizeof(float) * (size_t)c->numel()); }
// Handle of .grad (null if none has been accumulated).
FT_API void* ftc_grad(const void* h) { return H(T(h)->grad); }
FT_API void ftc_zero_grad(void* h) { T(h)->grad = nullptr; }
FT_API void* ftc_detach(const void* h) {
  auto t = std::make_shared<ft::TensorImpl>(*T(h));
  t->grad_fn = nullptr; t->grad = nullptr; t->requires_grad = false; t->hooks.clear(); t->post_acc_hooks.clear(); t->id = ft::g_next_id++;
  return H(t);
}
// Switches gradient recording on or off for the calling thread (no_grad); returns the previous setting.
FT_API int ftc_set_grad_enabled(int on) { const int prev = ft::g_grad_enabled; ft::g_grad_enabled = on != 0; return prev; }

FT_API void* ftc_add(const void* a, const void* b) { return H(ft::binary(ft::Bin::Add, T(a), T(b))); }
FT_API void* ftc_sub(const void* a, const void* b) { return H(ft::binary(ft::Bin::Sub, T(a), T(b))); }
FT_API void* ftc_mul(const void* a, const void* b) { return H(ft::binary(ft::Bin::Mul, T(a), T(b))); }
FT_API void* ftc_scale(const void* a, float s) { return H(ft::scale(T(a), s)); }
FT_API void* ftc_matmul(const void* a, const void* b) { return H(ft::matmul(T(a), T(b))); }
FT_API void* ftc_transpose(const void* a) { return H(ft::transpose(T(a))); }
FT_API void* ftc_relu(const void* a) { return H(ft::activation(ft::Act::Relu, T(a))); }
FT_API void* ftc_tanh(const void* a) { return H(ft::activation(ft::Act::Tanh, T(a))); }
FT_API void* ftc_sigmoid(const void* a) { return H(ft::activation(ft::Act::Sigmoid, T(a))); }
FT_API void* ftc_sum(const void* a) { return H(ft::sum(T(a), false)); }
FT_API void* ftc_mean(const void* a) { return H(ft::sum(T(a), true)); }
// x W^T + b (b may be null).
FT_API void* ftc_linear(const void* x, const void* w, const void* b) { return H(ft::linear(T(x), T(w), b ? T(b) : nullptr)); }
// Mean cross-entropy of logits [rows, classes] against `rows` int64 class indices.
FT_API void* ftc_cross_entropy(const void* logits, const int64_t* targets, int64_t rows) { return H(ft::cross_entropy(T(logits), targets, rows)); }

// Reverse-mode sweep from `root` (a scalar unless grad is given). threads <= 1: the serial engine; more: worker threads over the ready queue
// (same result bit for bit). Returns 0, or 1 if root does not require grad / is not a scalar without an explicit gradient.
FT_API int ftc_backward(void* root, const void* grad, int threads) {
  const Tensor& r = T(root);
  if (!r->requires_grad) { ft::g_last_error = "backward: the tensor does not require grad"; return 1; }
  Tensor g;
  if (grad) g = T(grad);
  else {
    if (r->numel() != 1) { ft::g_last_error = "backward: a gradient must be given for a non-scalar root"; return 1; }
    g = ft::make(r->shape, 1.f);
  }
  ft::backward(r, g, threads);
  return 0;
}

typedef void (*ftc_grad_hook)(void* user, float* grad, int64_t numel);
typedef void (*ftc_post_hook)(void* user, uint64_t tensor_id);
// fn(user, grad, numel) runs on every gradient that arrives at this tensor during backward and may rewrite it in place.
// (fn is passed as an untyped pointer so that the generated C header needs no typedef: void (*)(void* user, float* grad, int64_t numel).)
FT_API void ftc_register_hook(void* h, void* fn_ptr, void* user) {
  ftc_grad_hook fn = reinterpret_cast<ftc_grad_hook>(fn_ptr);
  T(h)->hooks.push_back([fn, user](ft::TensorImpl& g) { fn(user, g.data(), g.numel()); });
}
// fn(user, tensor_id) runs after a gradient has been accumulated into this leaf's .grad.
// (fn: void (*)(void* user, uint64_t tensor_id), passed as an untyped pointer.)
FT_API void ftc_register_post_accumulate_hook(void* h, void* fn_ptr, void* user) {
  ftc_post_hook fn = reinterpret_cast<ftc_post_hook>(fn_ptr);
  T(h)->post_acc_hooks.push_back([fn, user](ft::TensorImpl& t) { fn(user, t.id); });
}

// SGD over `n` parameter handles (the optimizer keeps references to them). Released with ftc_sgd_free.
FT_API void* ftc_sgd_new(void* const* params, int n, float lr, float momentum, float dampening, float weight_decay, int nesterov) {
  auto* s = new ft::Sgd();
  for (int i = 0; i < n; i++) s->params.push_back(T(params[i]));
  s->lr = lr; s->momentum = momentum; s->dampening = dampening; s->weight_decay = weight_decay; s->nesterov = nesterov != 0;
  return s;
}
FT_API void ftc_sgd_step(void* s) { static_cast<ft::Sgd*>(s)->step(); }
FT_API void ftc_sgd_set_lr(void* s, float lr) { static_cast<ft::Sgd*>(s)->lr = lr; }
FT_API void ftc_sgd_zero_grad(void* s) { for (auto& p : static_cast<ft::Sgd*>(s)->params) p->grad = nullptr; }
FT_API void ftc_sgd_free(void* s) { delete static_cast<ft::Sgd*>(s); }

// Element-wise operation `kind` (0 exp, 1 log, 2 sqrt, 3 gelu (erf form), 4 silu, 5 leaky relu with slope p, 6 power p, 7 abs, 8 square, 9 reciprocal).
FT_API void* ftc_unary(const void* a, int kind, float p) {
  if (kind < 0 || kind > 9) { ft::g_last_error = "unary: unknown kind"; return nullptr; }
  return H(ft::unary((ft::Un)kind, T(a), p));
}
FT_API void* ftc_div(const void* a, const void* b) { return H(ft::divide(T(a), T(b))); }
// A view with another shape (one entry may be -1); a non-contiguous input is copied first.
FT_API void* ftc_reshape(const void* a, const int64_t* shape, int ndim) { return H(ft::reshape(T(a), std::vector<int64_t>(shape, shape + ndim))); }
// Sum (mean = 0) or mean (mean = 1) along dimension dim (negative counts from the end).
FT_API void* ftc_sum_dim(const void* a, int dim, int keepdim, int mean) { return H(ft::sum_dim(T(a), dim, keepdim != 0, mean != 0)); }
// Softmax (log = 0) or log-softmax (log = 1) over the last dimension.
FT_API void* ftc_softmax(const void* a, int log) { return H(ft::softmax(T(a), log != 0)); }
// x [N, C, H, W], weight [O, C, kh, kw], bias [O] or null.
FT_API void* ftc_conv2d(const void* x, const void* w, const void* b, int sh, int sw, int ph, int pw) {
  return H(ft::conv2d(T(x), T(w), b ? T(b) : nullptr, sh, sw, ph, pw));
}
FT_API void* ftc_max_pool2d(const void* x, int k, int stride) { return H(ft::max_pool2d(T(x), k, stride)); }

FT_API void* ftc_adam_new(void* const* params, int n, float lr, float beta1, float beta2, float eps, float weight_decay, int decoupled) {
  auto* a = new ft::Adam();
  for (int i = 0; i < n; i++) a->params.push_back(T(params[i]));
  a->lr = lr; a->beta1 = beta1; a->beta2 = beta2; a->eps = eps; a->weight_decay = weight_decay; a->decoupled = decoupled != 0;
  return a;
}
FT_API void ftc_adam_step(void* s) { static_cast<ft::Adam*>(s)->step(); }
FT_API void ftc_adam_set_lr(void* s, float lr) { static_cast<ft::Adam*>(s)->lr = lr; }
FT_API void ftc_adam_zero_grad(void* s) { for (auto& p : static_cast<ft::Adam*>(s)->params) p->grad = nullptr; }
FT_API void ftc_adam_free(void* s) { delete static_cast<ft::Adam*>(s); }

// A view with the dimensions in the order dims (negative entries count from the end).
FT_API void* ftc_permute(const void* a, const int64_t* dims, int ndim) { return H(ft::permute(T(a), std::vector<int64_t>(dims, dims + ndim))); }
// [..., M, K] x [..., K, N] with equal leading dimensions.
FT_API void* ftc_bmm(const void* a, const void* b) { return H(ft::bmm(T(a), T(b))); }
// Normalisation over the last dimension; w and b ([last dim]) may be null.
FT_API void* ftc_layer_norm(const void* x, const void* w, const void* b, float eps) { return H(ft::layer_norm(T(x), w ? T(w) : nullptr, b ? T(b) : nullptr, eps)); }
// Rows ids (host int64, shape ids_shape) of table [rows, dim].
FT_API void* ftc_embedding(const void* table, const int64_t* ids, const int64_t* ids_shape, int ids_ndim) { return H(ft::embedding(T(table), ids, ids_shape, ids_ndim)); }
// A view of len consecutive entries of dimension dim starting at start.
FT_API void* ftc_narrow(const void* a, int dim, int64_t start, int64_t len) { return H(ft::narrow(T(a), dim, start, len)); }

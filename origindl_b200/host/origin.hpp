// C++ host layer above the C ABI (include/odl_b200.h): the reference's operator-level interface for the dense hot
// path, with the same names, argument meaning and error behaviour, running on one B200.
//
//   origin::Tensor / Parameter            include/origin/core/tensor.h:79-327, parameter.h:13-37
//   origin::Operator forward()/backward() include/origin/core/operator.h:12-125 (tape: src/core/tensor_impl.cpp:78-278)
//   origin::functional::mat_mul, relu, custom_linear, softmax_cross_entropy, conv2d, sum, broadcast_to, sum_to
//   origin::nn::Module, Linear, MLP       src/nn/module.cpp, src/nn/layers/linear.cpp, src/nn/models/mlp.cpp
//   origin::nn::Conv2d, BatchNorm1d, ReLU, SiLU, Flatten; origin::Sequential; functional::reshape, flatten
//                                         src/nn/layers/conv2d.cpp, batch_norm1d.cpp, relu.cpp, flatten.cpp, src/nn/sequential.cpp
//   functional::batch_norm, silu; nn::BatchNorm2d   src/operators/normalization/batch_norm.cpp, src/nn/layers/batch_norm2d.cpp
//   origin::Optimizer, SGD, Adam, WeightDecay   src/optim/*.cpp, include/origin/optim/hooks.h
//   origin::MemoryPool                    src/mat/origin/memory/memory_pool.cpp:37-176 (size-binned caching allocator)
//   origin::save / load / Checkpoint / load_checkpoint   src/io/model_io.cpp:114-273, src/io/checkpoint.cpp:15-226
//   origin::Dataset, DataLoader           include/origin/data/dataset.h, src/data/dataloader.cpp:11-146 (data set resident
//                                         in device memory, batches assembled by a gather kernel)
//
// Differences that are deliberate: tensors of this layer live on the device only (fp32 data, int32/int64 labels);
// nn::Linear and nn::MLP run the fused Linear(+ReLU) operator (one kernel forward, three backward) instead of
// mat_mul + broadcast_to + add + relu; optimizers update parameters in place; the loss stays on the device until
// item() is called.  Errors are std::invalid_argument / std::runtime_error, as the reference's THROW_* macros raise.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <any>
#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <queue>
#include <random>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "odl_b200.h"

namespace origin
{

// ------------------------------------------------------------------------------------------------ errors
inline void odl_check(int status)
{
    if (status == ODL_OK)
        return;
    const std::string msg = odl_last_error();
    if (status == ODL_ERR_INVALID_ARGUMENT || status == ODL_ERR_MISALIGNED || status == ODL_ERR_TOO_LARGE)
        throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

inline void cuda_check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess)
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

inline void init(int device = 0)
{
    odl_check(odl_init(device));
}

// Surfaces asynchronous kernel errors (bounded-wait time-outs, out-of-range labels) as exceptions.
inline void synchronize()
{
    odl_check(odl_device_status(nullptr));
}

// ------------------------------------------------------------------------------------------------ memory
// Caching device allocator with the reference's bin rule: powers of two from 256 B below 512 KB, then 1 / 4 / 16 MB,
// then multiples of 16 MB; freed blocks are kept for reuse until the cache exceeds its cap (512 MB by default).
class MemoryPool
{
  public:
    static MemoryPool &instance()
    {
        static MemoryPool p;
        return p;
    }
    static size_t bin_size(size_t bytes)
    {
        if (bytes <= 256)
            return 256;
        if (bytes <= (512u << 10))
        {
            size_t b = 256;
            while (b < bytes)
                b <<= 1;
            return b;
        }
        if (bytes <= (1u << 20))
            return 1u << 20;
        if (bytes <= (4u << 20))
            return 4u << 20;
        const size_t m16 = 16u << 20;
        return (bytes + m16 - 1) / m16 * m16;
    }
    void *malloc(size_t bytes, size_t *granted)
    {
        const size_t b = bin_size(bytes);
        *granted       = b;
        auto &lst      = free_[b];
        if (!lst.empty())
        {
            void *p = lst.back();
            lst.pop_back();
            cached_ -= b;
            ++hits_;
            return p;
        }
        void *p       = nullptr;
        cudaError_t e = cudaMalloc(&p, b);
        if (e != cudaSuccess)
        {
            release_cache();  // give cached blocks back and retry once
            e = cudaMalloc(&p, b);
        }
        cuda_check(e, "MemoryPool: cudaMalloc");
        ++misses_;
        return p;
    }
    void free(void *p, size_t granted)
    {
        if (!p)
            return;
        if (cached_ + granted > cap_)
        {
            cudaFree(p);  // synchronises the device, so no kernel can still be using the block
            return;
        }
        free_[granted].push_back(p);  // safe to hand out again: this layer issues everything on one stream
        cached_ += granted;
    }
    void release_cache()
    {
        for (auto &kv : free_)
            for (void *p : kv.second)
                cudaFree(p);
        free_.clear();
        cached_ = 0;
    }
    void set_cache_cap(size_t bytes) { cap_ = bytes; }
    size_t cached_bytes() const { return cached_; }
    size_t hits() const { return hits_; }
    size_t misses() const { return misses_; }
    ~MemoryPool() { release_cache(); }

  private:
    std::map<size_t, std::vector<void *>> free_;
    size_t cached_ = 0, cap_ = size_t(512) << 20, hits_ = 0, misses_ = 0;
};

struct Storage
{
    void *ptr      = nullptr;
    size_t granted = 0;
    explicit Storage(size_t bytes) { ptr = MemoryPool::instance().malloc(bytes == 0 ? 1 : bytes, &granted); }
    ~Storage() { MemoryPool::instance().free(ptr, granted); }
    Storage(const Storage &)            = delete;
    Storage &operator=(const Storage &) = delete;
};

// ------------------------------------------------------------------------------------------------ shape / dtype
class Shape
{
  public:
    Shape() = default;
    Shape(std::initializer_list<size_t> d) : d_(d) {}
    explicit Shape(std::vector<size_t> d) : d_(std::move(d)) {}
    size_t size() const { return d_.size(); }
    size_t operator[](size_t i) const { return d_.at(i); }
    size_t elements() const
    {
        size_t n = 1;
        for (size_t v : d_)
            n *= v;
        return n;
    }
    bool operator==(const Shape &o) const { return d_ == o.d_; }
    bool operator!=(const Shape &o) const { return d_ != o.d_; }
    std::string to_string() const
    {
        std::ostringstream s;
        s << "{";
        for (size_t i = 0; i < d_.size(); ++i)
            s << (i ? ", " : "") << d_[i];
        s << "}";
        return s.str();
    }
    const std::vector<size_t> &dims() const { return d_; }

  private:
    std::vector<size_t> d_;
};

enum class DataType
{
    kFloat32,
    kInt32,
    kInt64
};
inline size_t element_size(DataType t)
{
    return t == DataType::kInt64 ? 8 : 4;
}
template <typename T>
struct DataTypeTraits;
template <>
struct DataTypeTraits<float>
{
    static constexpr DataType type = DataType::kFloat32;
};
template <>
struct DataTypeTraits<int32_t>
{
    static constexpr DataType type = DataType::kInt32;
};
template <>
struct DataTypeTraits<int64_t>
{
    static constexpr DataType type = DataType::kInt64;
};

struct TensorOptions
{
    DataType dtype_     = DataType::kFloat32;
    bool requires_grad_ = false;
    TensorOptions() = default;
    TensorOptions(DataType t) : dtype_(t) {}
    TensorOptions &requires_grad(bool r)
    {
        requires_grad_ = r;
        return *this;
    }
};
inline TensorOptions dtype(DataType t)
{
    return TensorOptions(t);
}

// ------------------------------------------------------------------------------------------------ tensor
class Operator;
class Tensor;

struct TensorImpl
{
    Shape shape;
    DataType dtype = DataType::kFloat32;
    std::shared_ptr<Storage> storage;
    bool requires_grad = false;
    std::shared_ptr<TensorImpl> grad;
    std::shared_ptr<Operator> creator;
    int generation = 0;
};

class Tensor
{
  public:
    Tensor() = default;
    explicit Tensor(std::shared_ptr<TensorImpl> impl) : impl_(std::move(impl)) {}

    template <typename T>
    Tensor(const std::vector<T> &data, const Shape &shape, const TensorOptions &opt = TensorOptions(DataTypeTraits<T>::type))
    {
        if (data.size() != shape.elements())
            throw std::invalid_argument("Data size (" + std::to_string(data.size()) + ") does not match shape elements (" +
                                        std::to_string(shape.elements()) + ")");
        if (opt.dtype_ != DataTypeTraits<T>::type)
            throw std::invalid_argument("Tensor: data type of the values and of the options differ");
        alloc(shape, opt);
        cuda_check(cudaMemcpy(impl_->storage->ptr, data.data(), data.size() * sizeof(T), cudaMemcpyHostToDevice),
                   "Tensor: host to device copy");
    }
    template <typename T>
    Tensor(std::initializer_list<T> data, const Shape &shape, const TensorOptions &opt = TensorOptions(DataTypeTraits<T>::type))
        : Tensor(std::vector<T>(data), shape, opt)
    {
    }

    static Tensor empty(const Shape &shape, const TensorOptions &opt = TensorOptions())
    {
        Tensor t;
        t.alloc(shape, opt);
        return t;
    }
    static Tensor full(const Shape &shape, float value, const TensorOptions &opt = TensorOptions())
    {
        Tensor t = empty(shape, opt);
        if (opt.dtype_ != DataType::kFloat32)
            throw std::invalid_argument("Tensor::full: float32 only");
        if (shape.elements())
            odl_check(odl_fill(t.data_ptr<float>(), value, (int64_t)shape.elements(), nullptr));
        return t;
    }
    static Tensor zeros(const Shape &shape, const TensorOptions &opt = TensorOptions()) { return full(shape, 0.0f, opt); }
    static Tensor ones(const Shape &shape, const TensorOptions &opt = TensorOptions()) { return full(shape, 1.0f, opt); }
    // Standard normal values from a HOST generator with a fixed seed sequence (the reference's randn cannot be seeded).
    static Tensor randn(const Shape &shape, const TensorOptions &opt = TensorOptions(), uint64_t seed = 0)
    {
        static uint64_t counter = 0;
        std::mt19937_64 gen(seed ? seed : 0x9E3779B97F4A7C15ull + (++counter));
        std::normal_distribution<float> nd(0.0f, 1.0f);
        std::vector<float> v(shape.elements());
        for (auto &x : v)
            x = nd(gen);
        return Tensor(v, shape, opt);
    }

    bool defined() const { return impl_ != nullptr; }
    const Shape &shape() const { return must()->shape; }
    size_t ndim() const { return shape().size(); }
    size_t elements() const { return shape().elements(); }
    size_t numel() const { return elements(); }
    DataType dtype() const { return must()->dtype; }
    bool requires_grad() const { return must()->requires_grad; }
    template <typename T>
    T *data_ptr() const
    {
        return static_cast<T *>(must()->storage->ptr);
    }
    template <typename T>
    std::vector<T> to_vector() const
    {
        if (DataTypeTraits<T>::type != dtype())
            throw std::invalid_argument("to_vector: dtype mismatch");
        std::vector<T> v(elements());
        synchronize();
        cuda_check(cudaMemcpy(v.data(), must()->storage->ptr, v.size() * sizeof(T), cudaMemcpyDeviceToHost), "to_vector");
        return v;
    }
    template <typename T>
    T item() const
    {
        if (elements() != 1)
            throw std::runtime_error("item() requires a tensor with exactly one element, got shape " + shape().to_string());
        return to_vector<T>()[0];
    }
    Tensor reshape(const Shape &s) const
    {
        if (s.elements() != elements())
            throw std::invalid_argument("reshape: cannot reshape " + shape().to_string() + " to " + s.to_string());
        auto impl           = std::make_shared<TensorImpl>(*must());
        impl->shape         = s;
        impl->grad          = nullptr;
        impl->creator       = nullptr;
        impl->requires_grad = false;
        return Tensor(impl);
    }
    Tensor detach() const { return reshape(shape()); }
    Tensor clone() const
    {
        Tensor t = empty(shape(), TensorOptions(dtype()));
        cuda_check(cudaMemcpyAsync(t.must()->storage->ptr, must()->storage->ptr, elements() * element_size(dtype()),
                                   cudaMemcpyDeviceToDevice, nullptr),
                   "clone");
        return t;
    }

    Tensor grad() const
    {
        if (!must()->grad)
            throw std::runtime_error("grad(): tensor has no gradient");
        return Tensor(must()->grad);
    }
    bool has_grad() const { return impl_ && impl_->grad != nullptr; }
    void clear_grad() { must()->grad = nullptr; }
    void accumulate_grad(const Tensor &g);
    void backward();

    std::shared_ptr<TensorImpl> impl() const { return impl_; }

  protected:
    void alloc(const Shape &shape, const TensorOptions &opt)
    {
        impl_                = std::make_shared<TensorImpl>();
        impl_->shape         = shape;
        impl_->dtype         = opt.dtype_;
        impl_->requires_grad = opt.requires_grad_;
        impl_->storage       = std::make_shared<Storage>(shape.elements() * element_size(opt.dtype_));
    }
    TensorImpl *must() const
    {
        if (!impl_)
            throw std::runtime_error("operation on an undefined Tensor");
        return impl_.get();
    }
    std::shared_ptr<TensorImpl> impl_;
};

class Parameter : public Tensor
{
  public:
    Parameter() = default;
    Parameter(const Tensor &t) : Tensor(t) {}
};

// ------------------------------------------------------------------------------------------------ operator + tape
struct Config
{
    static bool &enable_backprop()
    {
        static bool v = true;
        return v;
    }
};
struct NoGradGuard  // include/origin/core/config.h: no_grad()
{
    bool prev;
    NoGradGuard() : prev(Config::enable_backprop()) { Config::enable_backprop() = false; }
    ~NoGradGuard() { Config::enable_backprop() = prev; }
};

class Operator : public std::enable_shared_from_this<Operator>
{
  public:
    virtual ~Operator() = default;
    virtual std::vector<Tensor> forward(const std::vector<Tensor> &xs)   = 0;
    virtual std::vector<Tensor> backward(const std::vector<Tensor> &gys) = 0;

    // Runs forward and, when any input requires a gradient, records the node on the tape
    // (include/origin/core/operator.h:21-59, src/operators/operator.cpp:9-36).
    std::vector<Tensor> operator()(const std::vector<Tensor> &xs)
    {
        std::vector<Tensor> ys = forward(xs);
        bool any               = false;
        for (const Tensor &x : xs)
            any = any || (x.defined() && x.requires_grad());
        if (Config::enable_backprop() && any)
        {
            inputs_     = xs;
            generation_ = 0;
            for (const Tensor &x : xs)
                generation_ = std::max(generation_, x.impl()->generation);
            for (Tensor &y : ys)
            {
                y.impl()->requires_grad = true;
                y.impl()->creator       = shared_from_this();
                y.impl()->generation    = generation_ + 1;
                outputs_.push_back(y.impl());
            }
        }
        return ys;
    }
    Tensor call1(const std::vector<Tensor> &xs) { return (*this)(xs)[0]; }

    std::vector<Tensor> inputs_;
    std::vector<std::weak_ptr<TensorImpl>> outputs_;
    int generation_ = 0;
};

inline void Tensor::accumulate_grad(const Tensor &g)
{
    if (g.shape() != shape())
        throw std::invalid_argument("accumulate_grad: gradient shape " + g.shape().to_string() + " != " + shape().to_string());
    if (!must()->grad)
        must()->grad = g.impl();  // the first gradient shares the produced tensor (src/core/tensor_impl.cpp:187-191)
    else
        odl_check(odl_binary(0, Tensor(must()->grad).data_ptr<float>(), g.data_ptr<float>(),
                             Tensor(must()->grad).data_ptr<float>(), (int64_t)elements(), nullptr));
}

inline void Tensor::backward()
{
    if (!must()->grad)
        must()->grad = Tensor::ones(shape()).impl();
    auto cmp = [](const std::shared_ptr<Operator> &a, const std::shared_ptr<Operator> &b) {
        return a->generation_ < b->generation_;
    };
    std::priority_queue<std::shared_ptr<Operator>, std::vector<std::shared_ptr<Operator>>, decltype(cmp)> todo(cmp);
    std::set<Operator *> seen;
    std::vector<std::shared_ptr<Operator>> visited;
    auto push = [&](const std::shared_ptr<Operator> &f) {
        if (f && seen.insert(f.get()).second)
        {
            todo.push(f);
            visited.push_back(f);
        }
    };
    push(must()->creator);
    while (!todo.empty())
    {
        auto f = todo.top();
        todo.pop();
        std::vector<Tensor> gys;
        for (auto &w : f->outputs_)
        {
            auto o = w.lock();
            gys.push_back(o && o->grad ? Tensor(o->grad) : Tensor());
        }
        std::vector<Tensor> gxs = f->backward(gys);
        if (gxs.size() != f->inputs_.size())
            throw std::runtime_error("backward: operator returned " + std::to_string(gxs.size()) + " gradients for " +
                                     std::to_string(f->inputs_.size()) + " inputs");
        for (size_t i = 0; i < gxs.size(); ++i)
        {
            Tensor &x = f->inputs_[i];
            if (!x.defined() || !x.requires_grad() || !gxs[i].defined())
                continue;
            x.accumulate_grad(gxs[i]);
            push(x.impl()->creator);
        }
    }
    // tear the graph down: intermediates lose their creator and gradient, leaves keep theirs (tensor_impl.cpp:205-277)
    for (auto &f : visited)
    {
        for (auto &w : f->outputs_)
            if (auto o = w.lock())
            {
                o->creator = nullptr;
                if (o.get() != impl_.get())
                    o->grad = nullptr;
            }
        f->inputs_.clear();
    }
}

// ------------------------------------------------------------------------------------------------ operators
namespace detail
{
inline int precision()
{
    static const int p = [] {
        const char *e = std::getenv("ORIGIN_MATMUL_PRECISION");
        return (e && std::string(e) == "tf32") ? ODL_PRECISION_TF32 : ODL_PRECISION_3XTF32;
    }();
    return p;
}
inline void need_f32(const Tensor &t, const char *who)
{
    if (t.dtype() != DataType::kFloat32)
        throw std::invalid_argument(std::string(who) + ": float32 tensors only on this path");
}
inline int64_t i64(size_t v)
{
    return static_cast<int64_t>(v);
}
}  // namespace detail

namespace functional
{

// y = x . w for 2-D, 3-D x 2-D and 3-D x 3-D operands (src/operators/math/mat_mul.cpp:12-182).
class MatMul : public Operator
{
  public:
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != 2)
            throw std::runtime_error("MatMul operator requires exactly 2 inputs, but got " + std::to_string(xs.size()));
        const Tensor &a = xs[0], &b = xs[1];
        detail::need_f32(a, "mat_mul");
        detail::need_f32(b, "mat_mul");
        const Shape &as = a.shape(), &bs = b.shape();
        if (as.size() == 2 && bs.size() == 2)
        {
            if (as[1] != bs[0])
                throw std::invalid_argument("Matrix dimensions must be compatible for multiplication. A shape: " +
                                            as.to_string() + ", B shape: " + bs.to_string());
            Tensor y = Tensor::empty(Shape{as[0], bs[1]});
            odl_check(odl_matmul(a.data_ptr<float>(), b.data_ptr<float>(), y.data_ptr<float>(), detail::i64(as[0]),
                                 detail::i64(bs[1]), detail::i64(as[1]), 1, 0, detail::precision(), nullptr));
            return {y};
        }
        if (as.size() == 3 && (bs.size() == 2 || bs.size() == 3))
        {
            const bool b3 = bs.size() == 3;
            if ((b3 && (as[0] != bs[0] || as[2] != bs[1])) || (!b3 && as[2] != bs[0]))
                throw std::invalid_argument("Matrix dimensions must be compatible for multiplication. A shape: " +
                                            as.to_string() + ", B shape: " + bs.to_string());
            const size_t n = b3 ? bs[2] : bs[1];
            Tensor y       = Tensor::empty(Shape{as[0], as[1], n});
            odl_check(odl_matmul(a.data_ptr<float>(), b.data_ptr<float>(), y.data_ptr<float>(), detail::i64(as[1]),
                                 detail::i64(n), detail::i64(as[2]), detail::i64(as[0]), b3 ? 1 : 0, detail::precision(),
                                 nullptr));
            return {y};
        }
        throw std::invalid_argument("Matrix multiplication requires compatible dimensions. A shape: " + as.to_string() +
                                    ", B shape: " + bs.to_string());
    }
    // gx = gy . w^T, gw = x^T . gy without materialised transposes (mat_mul.cpp:123-182)
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        const Tensor &x = inputs_[0], &w = inputs_[1], &gy = gys[0];
        if (x.ndim() != 2 || w.ndim() != 2)
            throw std::runtime_error("MatMul::backward: only the 2-D form is differentiated on this path");
        const int64_t M = detail::i64(x.shape()[0]), K = detail::i64(x.shape()[1]), N = detail::i64(w.shape()[1]);
        Tensor gx = Tensor::empty(x.shape()), gw = Tensor::empty(w.shape());
        odl_check(odl_gemm_ex(0, 1, M, K, N, gy.data_ptr<float>(), nullptr, N, w.data_ptr<float>(), nullptr, N,
                              gx.data_ptr<float>(), nullptr, K, nullptr, nullptr, 0, nullptr, 0, detail::precision(), nullptr));
        odl_check(odl_gemm_ex(1, 0, K, N, M, x.data_ptr<float>(), nullptr, K, gy.data_ptr<float>(), nullptr, N,
                              gw.data_ptr<float>(), nullptr, N, nullptr, nullptr, 0, nullptr, 0, detail::precision(), nullptr));
        return {gx, gw};
    }
};

// Same-shape element-wise add / subtract / multiply (src/operators/math/{add,sub,mul}.cpp).
class Binary : public Operator
{
  public:
    explicit Binary(int op) : op_(op) {}
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != 2)
            throw std::runtime_error("binary operator requires exactly 2 inputs");
        if (xs[0].shape() != xs[1].shape())
            throw std::invalid_argument("binary operator: shapes differ (" + xs[0].shape().to_string() + " vs " +
                                        xs[1].shape().to_string() + "); broadcast_to the smaller operand first");
        Tensor y = Tensor::empty(xs[0].shape());
        odl_check(odl_binary(op_, xs[0].data_ptr<float>(), xs[1].data_ptr<float>(), y.data_ptr<float>(),
                             detail::i64(y.elements()), nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        const Tensor &gy = gys[0];
        const int64_t n  = detail::i64(gy.elements());
        if (op_ == 0)
            return {gy, gy};
        if (op_ == 1)
        {
            Tensor g1 = Tensor::empty(gy.shape());
            odl_check(odl_scale(gy.data_ptr<float>(), -1.0f, g1.data_ptr<float>(), n, nullptr));
            return {gy, g1};
        }
        Tensor g0 = Tensor::empty(gy.shape()), g1 = Tensor::empty(gy.shape());
        odl_check(odl_binary(2, gy.data_ptr<float>(), inputs_[1].data_ptr<float>(), g0.data_ptr<float>(), n, nullptr));
        odl_check(odl_binary(2, gy.data_ptr<float>(), inputs_[0].data_ptr<float>(), g1.data_ptr<float>(), n, nullptr));
        return {g0, g1};
    }

  private:
    int op_;
};

class Scale : public Operator  // tensor * scalar (src/operators/math/mul.cpp:113-117)
{
  public:
    explicit Scale(float a) : a_(a) {}
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        Tensor y = Tensor::empty(xs[0].shape());
        odl_check(odl_scale(xs[0].data_ptr<float>(), a_, y.data_ptr<float>(), detail::i64(y.elements()), nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        Tensor g = Tensor::empty(gys[0].shape());
        odl_check(odl_scale(gys[0].data_ptr<float>(), a_, g.data_ptr<float>(), detail::i64(g.elements()), nullptr));
        return {g};
    }

  private:
    float a_;
};

// {1,N} -> {M,N} (src/operators/math/broadcast_to.cpp:10-46); backward is sum_to.
class BroadcastTo : public Operator
{
  public:
    explicit BroadcastTo(Shape s) : shape_(std::move(s)) {}
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        const Tensor &x = xs[0];
        if (x.shape() == shape_)
            return {x};
        if (shape_.size() != 2 || x.elements() != shape_[1])
            throw std::invalid_argument("broadcast_to: only {1,N} or {N} -> {M,N} on this path, got " +
                                        x.shape().to_string() + " -> " + shape_.to_string());
        Tensor y = Tensor::zeros(shape_);
        odl_check(odl_add_bias(y.data_ptr<float>(), x.data_ptr<float>(), y.data_ptr<float>(), detail::i64(shape_[0]),
                               detail::i64(shape_[1]), nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        const Tensor &x = inputs_[0];
        if (x.shape() == shape_)
            return {gys[0]};
        Tensor g = Tensor::empty(x.shape());
        odl_check(odl_sum_to_row(gys[0].data_ptr<float>(), g.data_ptr<float>(), detail::i64(shape_[0]),
                                 detail::i64(shape_[1]), nullptr));
        return {g};
    }

  private:
    Shape shape_;
};

class Sum : public Operator  // sum of all elements -> 0-dim (src/operators/math/sum.cpp, axis = -1)
{
  public:
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        Tensor y = Tensor::empty(Shape{});
        odl_check(odl_sum_all(xs[0].data_ptr<float>(), y.data_ptr<float>(), detail::i64(xs[0].elements()), nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        const float g = gys[0].item<float>();
        return {Tensor::full(inputs_[0].shape(), g)};
    }
};

class ReLU : public Operator  // src/operators/activation/relu.cpp:13-54
{
  public:
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != 1)
            throw std::runtime_error("ReLU operator requires exactly 1 input, but got " + std::to_string(xs.size()));
        Tensor y = Tensor::empty(xs[0].shape());
        odl_check(odl_relu_forward(xs[0].data_ptr<float>(), y.data_ptr<float>(), detail::i64(y.elements()), nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        Tensor g = Tensor::empty(gys[0].shape());
        odl_check(odl_relu_backward(gys[0].data_ptr<float>(), inputs_[0].data_ptr<float>(), g.data_ptr<float>(),
                                    detail::i64(g.elements()), nullptr));
        return {g};
    }
};

class SiLU : public Operator  // src/operators/activation/silu.cpp
{
  public:
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != 1)
            throw std::runtime_error("SiLU operator requires exactly 1 input, but got " + std::to_string(xs.size()));
        Tensor y = Tensor::empty(xs[0].shape());
        odl_check(odl_silu_forward(xs[0].data_ptr<float>(), y.data_ptr<float>(), detail::i64(y.elements()), nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        Tensor g = Tensor::empty(gys[0].shape());
        odl_check(odl_silu_backward(gys[0].data_ptr<float>(), inputs_[0].data_ptr<float>(), g.data_ptr<float>(),
                                    detail::i64(g.elements()), nullptr));
        return {g};
    }
};

// Inputs (x, gamma, beta, running_mean, running_var), x {N,C} (num_dims 2) or {N,C,H,W} (num_dims 4)
// (src/operators/normalization/batch_norm.cpp:18-118).  Differences from the reference operator, all deliberate:
// one output (the batch statistics are read with mean() / var()), so that backward also works after a TRAINING-mode
// forward -- the reference returns three outputs there and its own backward then throws; no x_norm tensor is kept;
// `act` fuses a ReLU / SiLU; `update_running` applies nn::BatchNorm2d's running-statistics rule inside the kernel.
class BatchNorm : public Operator
{
  public:
    BatchNorm(bool training, float eps, float momentum, int num_dims, int act = ODL_ACT_NONE, bool update_running = false)
        : training_(training), eps_(eps), momentum_(momentum), num_dims_(num_dims), act_(act), update_(update_running)
    {
    }
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != 5)
            throw std::runtime_error("BatchNorm operator requires exactly 5 inputs (x, gamma, beta, running_mean, "
                                     "running_var), but got " + std::to_string(xs.size()));
        const Tensor &x = xs[0];
        if (num_dims_ != 2 && num_dims_ != 4)
            throw std::invalid_argument("batch_norm: num_dims must be 2 or 4, but got " + std::to_string(num_dims_));
        if (x.ndim() != (size_t)num_dims_)
            throw std::invalid_argument("batch_norm: x must have " + std::to_string(num_dims_) +
                                        " dimensions, but got shape " + x.shape().to_string());
        const size_t C = x.shape()[1];
        for (int i = 1; i < 5; ++i)
            if (xs[i].shape() != Shape{C})
                throw std::invalid_argument("batch_norm: gamma, beta, running_mean, running_var must have shape (" +
                                            std::to_string(C) + ")");
        detail::need_f32(x, "batch_norm");
        const int64_t hw = num_dims_ == 4 ? detail::i64(x.shape()[2] * x.shape()[3]) : 1;
        Tensor y = Tensor::empty(x.shape());
        mean_    = Tensor::empty(Shape{C});
        var_     = Tensor::empty(Shape{C});
        const bool pass_running = !training_ || update_;
        odl_check(odl_batch_norm_forward(x.data_ptr<float>(), xs[1].data_ptr<float>(), xs[2].data_ptr<float>(),
                                         pass_running ? xs[3].data_ptr<float>() : nullptr,
                                         pass_running ? xs[4].data_ptr<float>() : nullptr, training_ ? 1 : 0, eps_, momentum_,
                                         detail::i64(x.shape()[0]), detail::i64(C), hw, act_, y.data_ptr<float>(),
                                         mean_.data_ptr<float>(), var_.data_ptr<float>(), nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        if (gys.size() != 1)
            throw std::runtime_error("BatchNorm backward requires exactly 1 gradient, but got " + std::to_string(gys.size()));
        const Tensor &x = inputs_[0];
        const size_t C  = x.shape()[1];
        const int64_t hw = num_dims_ == 4 ? detail::i64(x.shape()[2] * x.shape()[3]) : 1;
        Tensor gx = Tensor::empty(x.shape()), dgamma = Tensor::empty(Shape{C}), dbeta = Tensor::empty(Shape{C});
        odl_check(odl_batch_norm_backward(gys[0].data_ptr<float>(), x.data_ptr<float>(), inputs_[1].data_ptr<float>(),
                                          inputs_[2].data_ptr<float>(), mean_.data_ptr<float>(), var_.data_ptr<float>(), eps_,
                                          detail::i64(x.shape()[0]), detail::i64(C), hw, act_, gx.data_ptr<float>(),
                                          dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), nullptr));
        return {gx, dgamma, dbeta, Tensor(), Tensor()};
    }
    const Tensor &mean() const { return mean_; }  // statistics the last forward normalised with
    const Tensor &var() const { return var_; }

  private:
    bool training_;
    float eps_, momentum_;
    int num_dims_, act_;
    bool update_;
    Tensor mean_, var_;
};

// y = relu?(x . op(W) + b) as ONE kernel; backward = dX, dW, db with the ReLU mask and the column sums fused.
// w_layout ODL_W_OUT_IN is LinearOp / custom_linear (src/operators/custom/linear.cpp), whose backward the reference
// leaves unimplemented; ODL_W_IN_OUT is nn::Linear's weight (src/nn/layers/linear.cpp).
class LinearOp : public Operator
{
  public:
    LinearOp(int in_features, int out_features, bool use_bias, int w_layout = ODL_W_OUT_IN, bool relu = false)
        : in_(in_features), out_(out_features), bias_(use_bias), layout_(w_layout), relu_(relu)
    {
    }
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != (bias_ ? 3u : 2u))
            throw std::runtime_error("LinearOp requires " + std::to_string(bias_ ? 3 : 2) + " inputs, but got " +
                                     std::to_string(xs.size()));
        const Tensor &x = xs[0], &w = xs[1];
        detail::need_f32(x, "custom_linear");
        const size_t feat = x.ndim() >= 1 ? x.shape()[x.ndim() - 1] : 0;
        if (x.ndim() < 2 && !(x.ndim() == 1))
            throw std::invalid_argument("custom_linear: input must have at least 1 dimension");
        const size_t rows = x.elements() / (feat ? feat : 1);
        if ((int)feat != in_)
            throw std::invalid_argument("custom_linear: input feature size " + std::to_string(feat) +
                                        " does not match in_features " + std::to_string(in_));
        const Shape want = layout_ == ODL_W_OUT_IN ? Shape{(size_t)out_, (size_t)in_} : Shape{(size_t)in_, (size_t)out_};
        if (w.shape() != want)
            throw std::invalid_argument("custom_linear: weight shape " + w.shape().to_string() + " != " + want.to_string());
        if (bias_ && xs[2].elements() != (size_t)out_)
            throw std::invalid_argument("custom_linear: bias size mismatch");
        Tensor y = Tensor::empty(Shape{rows, (size_t)out_});
        odl_check(odl_linear_forward(x.data_ptr<float>(), nullptr, w.data_ptr<float>(), nullptr,
                                     bias_ ? xs[2].data_ptr<float>() : nullptr, y.data_ptr<float>(), nullptr,
                                     detail::i64(rows), out_, in_, layout_, relu_ ? 1 : 0, detail::precision(), nullptr));
        y_ = relu_ ? y.detach() : Tensor();
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        const Tensor &x = inputs_[0], &w = inputs_[1];
        const int64_t rows = detail::i64(x.elements() / (size_t)in_);
        Tensor gx = Tensor::empty(x.shape()), gw = Tensor::empty(w.shape());
        Tensor gb = bias_ ? Tensor::empty(inputs_[2].shape()) : Tensor();
        odl_check(odl_linear_backward(x.data_ptr<float>(), nullptr, w.data_ptr<float>(), nullptr, gys[0].data_ptr<float>(),
                                      relu_ ? y_.data_ptr<float>() : nullptr, gx.data_ptr<float>(), gw.data_ptr<float>(),
                                      bias_ ? gb.data_ptr<float>() : nullptr, rows, out_, in_, layout_, detail::precision(),
                                      nullptr));
        if (bias_)
            return {gx, gw, gb};
        return {gx, gw};
    }

  private:
    int in_, out_;
    bool bias_;
    int layout_;
    bool relu_;
    Tensor y_;
};

// loss = -(1/N) sum log(softmax(x)[i, t_i] + 1e-8) kept on the device (src/operators/loss/softmax_cross_entropy.cpp).
class SoftmaxCrossEntropy : public Operator
{
  public:
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != 2)
            throw std::runtime_error("SoftmaxCrossEntropy operator requires exactly 2 inputs (x and target), but got " +
                                     std::to_string(xs.size()));
        const Tensor &x = xs[0], &t = xs[1];
        if (x.ndim() != 2)
            throw std::invalid_argument("SoftmaxCrossEntropy expects x to be 2D (N, C), but got shape " + x.shape().to_string());
        if (t.ndim() != 1)
            throw std::invalid_argument("SoftmaxCrossEntropy expects target to be 1D (N,), but got shape " +
                                        t.shape().to_string());
        if (x.shape()[0] != t.shape()[0])
            throw std::invalid_argument("SoftmaxCrossEntropy: batch size mismatch. x has " + std::to_string(x.shape()[0]) +
                                        " samples, target has " + std::to_string(t.shape()[0]) + " samples");
        if (t.dtype() == DataType::kFloat32)
            throw std::invalid_argument("SoftmaxCrossEntropy: target must be int32 or int64");
        Tensor loss = Tensor::empty(Shape{});
        odl_check(odl_softmax_cross_entropy(x.data_ptr<float>(), t.data_ptr<void>(), t.dtype() == DataType::kInt64,
                                            detail::i64(x.shape()[0]), detail::i64(x.shape()[1]), loss.data_ptr<float>(),
                                            nullptr, 1.0f, nullptr));
        synchronize();  // an out-of-range label throws here, where the reference throws from gather
        return {loss};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        const Tensor &x = inputs_[0], &t = inputs_[1];
        const float gy  = gys[0].item<float>();
        Tensor gx       = Tensor::empty(x.shape());
        odl_check(odl_softmax_cross_entropy(x.data_ptr<float>(), t.data_ptr<void>(), t.dtype() == DataType::kInt64,
                                            detail::i64(x.shape()[0]), detail::i64(x.shape()[1]), nullptr,
                                            gx.data_ptr<float>(), gy, nullptr));
        return {gx, Tensor()};
    }
};

class Conv2dOp : public Operator  // src/operators/conv/conv2d.cpp:14-89
{
  public:
    Conv2dOp(int stride, int pad, bool use_bias, int gy_layout = 0)
        : stride_(stride), pad_(pad), bias_(use_bias), gy_layout_(gy_layout)
    {
    }
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        const Tensor &x = xs[0], &w = xs[1];
        if (x.ndim() != 4)
            throw std::invalid_argument("conv2d: x must be 4D (N, C, H, W), but got shape " + x.shape().to_string());
        if (w.ndim() != 4)
            throw std::invalid_argument("conv2d: W must be 4D (OC, C, KH, KW), but got shape " + w.shape().to_string());
        if (x.shape()[1] != w.shape()[1])
            throw std::invalid_argument("conv2d: channel mismatch - x has " + std::to_string(x.shape()[1]) +
                                        " channels, but W expects " + std::to_string(w.shape()[1]) + " channels");
        const int64_t N = detail::i64(x.shape()[0]), C = detail::i64(x.shape()[1]), H = detail::i64(x.shape()[2]),
                      W = detail::i64(x.shape()[3]), OC = detail::i64(w.shape()[0]);
        const int KH = (int)w.shape()[2], KW = (int)w.shape()[3];
        const int OH = (int)((H + 2 * pad_ - KH) / stride_ + 1), OW = (int)((W + 2 * pad_ - KW) / stride_ + 1);
        if (OH <= 0 || OW <= 0)
            throw std::invalid_argument("conv2d: invalid output size OH=" + std::to_string(OH) + ", OW=" + std::to_string(OW));
        if (bias_ && (xs[2].ndim() != 1 || xs[2].shape()[0] != (size_t)OC))
            throw std::invalid_argument("conv2d: b must be 1D with size " + std::to_string(OC));
        Tensor y = Tensor::empty(Shape{(size_t)N, (size_t)OC, (size_t)OH, (size_t)OW});
        odl_check(odl_conv2d_forward(x.data_ptr<float>(), w.data_ptr<float>(), bias_ ? xs[2].data_ptr<float>() : nullptr,
                                     y.data_ptr<float>(), N, C, H, W, OC, KH, KW, stride_, pad_, 0, detail::precision(),
                                     nullptr));
        return {y};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override
    {
        const Tensor &x = inputs_[0], &w = inputs_[1];
        Tensor gx = Tensor::empty(x.shape()), gw = Tensor::empty(w.shape());
        Tensor gb = bias_ ? Tensor::empty(inputs_[2].shape()) : Tensor();
        odl_check(odl_conv2d_backward(gys[0].data_ptr<float>(), x.data_ptr<float>(), w.data_ptr<float>(),
                                      gx.data_ptr<float>(), gw.data_ptr<float>(), bias_ ? gb.data_ptr<float>() : nullptr,
                                      detail::i64(x.shape()[0]), detail::i64(x.shape()[1]), detail::i64(x.shape()[2]),
                                      detail::i64(x.shape()[3]), detail::i64(w.shape()[0]), (int)w.shape()[2],
                                      (int)w.shape()[3], stride_, pad_, gy_layout_, detail::precision(), nullptr));
        if (bias_)
            return {gx, gw, gb};
        return {gx, gw};
    }

  private:
    int stride_, pad_;
    bool bias_;
    int gy_layout_;
};

// ---- free functions with the reference's names
inline Tensor mat_mul(const Tensor &x, const Tensor &w) { return std::make_shared<MatMul>()->call1({x, w}); }
inline Tensor relu(const Tensor &x) { return std::make_shared<ReLU>()->call1({x}); }
inline Tensor silu(const Tensor &x) { return std::make_shared<SiLU>()->call1({x}); }
inline Tensor batch_norm(const Tensor &x, const Tensor &gamma, const Tensor &beta, const Tensor &running_mean,
                         const Tensor &running_var, bool training, float eps = 1e-5f, float momentum = 0.1f,
                         int num_dims = 4)
{
    return std::make_shared<BatchNorm>(training, eps, momentum, num_dims)->call1({x, gamma, beta, running_mean, running_var});
}
inline Tensor sum(const Tensor &x) { return std::make_shared<Sum>()->call1({x}); }
inline Tensor broadcast_to(const Tensor &x, const Shape &s) { return std::make_shared<BroadcastTo>(s)->call1({x}); }
inline Tensor sum_to(const Tensor &x, const Shape &s)
{
    if (x.shape() == s)
        return x;
    if (x.ndim() != 2 || s.elements() != x.shape()[1])
        throw std::invalid_argument("sum_to: only {M,N} -> {1,N} on this path");
    Tensor y = Tensor::empty(s);
    odl_check(odl_sum_to_row(x.data_ptr<float>(), y.data_ptr<float>(), detail::i64(x.shape()[0]), detail::i64(x.shape()[1]),
                             nullptr));
    return y;
}
inline Tensor custom_linear(const Tensor &x, const Tensor &weight, const Tensor &bias, int in_features, int out_features,
                            bool use_bias)
{
    auto op = std::make_shared<LinearOp>(in_features, out_features, use_bias);
    return use_bias ? op->call1({x, weight, bias}) : op->call1({x, weight});
}
inline Tensor custom_linear(const Tensor &x, const Tensor &weight, int in_features, int out_features)
{
    return std::make_shared<LinearOp>(in_features, out_features, false)->call1({x, weight});
}
// A view of the same storage under another shape; the gradient is the upstream gradient under the input's shape
// (src/operators/shape/reshape.cpp; flatten: src/operators/shape/flatten.cpp).  No kernel runs in either direction.
class Reshape : public Operator
{
  public:
    explicit Reshape(Shape shape) : shape_(std::move(shape)) {}
    std::vector<Tensor> forward(const std::vector<Tensor> &xs) override
    {
        if (xs.size() != 1)
            throw std::runtime_error("Reshape operator requires exactly 1 input, but got " + std::to_string(xs.size()));
        return {xs[0].reshape(shape_)};
    }
    std::vector<Tensor> backward(const std::vector<Tensor> &gys) override { return {gys[0].reshape(inputs_[0].shape())}; }

  private:
    Shape shape_;
};

inline Tensor reshape(const Tensor &x, const Shape &shape) { return std::make_shared<Reshape>(shape)->call1({x}); }
// Dimensions start_dim..end_dim (negative values count from the end) collapse into one (functional::flatten).
inline Tensor flatten(const Tensor &x, int start_dim = 1, int end_dim = -1)
{
    const int nd = static_cast<int>(x.ndim());
    const int a = start_dim < 0 ? start_dim + nd : start_dim, b = end_dim < 0 ? end_dim + nd : end_dim;
    if (a < 0 || b >= nd || a > b)
        throw std::invalid_argument("flatten: invalid dimensions [" + std::to_string(start_dim) + ", " +
                                    std::to_string(end_dim) + "] for shape " + x.shape().to_string());
    std::vector<size_t> d;
    size_t merged = 1;
    for (int i = 0; i < nd; ++i)
    {
        if (i < a || i > b)
            d.push_back(x.shape()[i]);
        else
        {
            merged *= x.shape()[i];
            if (i == b)
                d.push_back(merged);
        }
    }
    return reshape(x, Shape(d));
}
inline Tensor softmax_cross_entropy(const Tensor &x, const Tensor &target)
{
    return std::make_shared<SoftmaxCrossEntropy>()->call1({x, target});
}
inline Tensor conv2d(const Tensor &x, const Tensor &W, const Tensor *b = nullptr, int stride = 1, int pad = 0)
{
    auto op = std::make_shared<Conv2dOp>(stride, pad, b != nullptr);
    return b ? op->call1({x, W, *b}) : op->call1({x, W});
}

}  // namespace functional

inline Tensor operator+(const Tensor &a, const Tensor &b) { return std::make_shared<functional::Binary>(0)->call1({a, b}); }
inline Tensor operator-(const Tensor &a, const Tensor &b) { return std::make_shared<functional::Binary>(1)->call1({a, b}); }
inline Tensor operator*(const Tensor &a, const Tensor &b) { return std::make_shared<functional::Binary>(2)->call1({a, b}); }
inline Tensor operator*(const Tensor &a, float s) { return std::make_shared<functional::Scale>(s)->call1({a}); }

// ------------------------------------------------------------------------------------------------ nn
namespace nn
{

class Module
{
  public:
    virtual ~Module() = default;
    virtual Tensor forward(const Tensor &x) = 0;
    Tensor operator()(const Tensor &x) { return forward(x); }
    virtual std::vector<Parameter *> parameters()
    {
        std::vector<Parameter *> out;
        for (auto &kv : params_)
            out.push_back(kv.second);
        for (auto &kv : modules_)
            for (Parameter *p : kv.second->parameters())
                out.push_back(p);
        return out;
    }
    std::map<std::string, Parameter *> named_parameters(const std::string &prefix = "")
    {
        std::map<std::string, Parameter *> out;
        for (auto &kv : params_)
            out[prefix + kv.first] = kv.second;
        for (auto &kv : modules_)
            for (auto &sub : kv.second->named_parameters(prefix + kv.first + "."))
                out[sub.first] = sub.second;
        return out;
    }
    void zero_grad()
    {
        for (Parameter *p : parameters())
            p->clear_grad();
    }
    // The parameters themselves (shared storage) keyed by dotted name (src/nn/module.cpp:118-128).
    using StateDict = std::unordered_map<std::string, Tensor>;
    virtual StateDict state_dict()
    {
        StateDict sd;
        for (auto &kv : named_parameters())
            sd[kv.first] = static_cast<const Tensor &>(*kv.second);
        return sd;
    }
    // src/nn/module.cpp:130-168: a shape mismatch always throws; missing / unexpected names throw in strict mode.
    // The parameter takes the VALUES of the loaded tensor (a device copy that requires grad).
    virtual void load_state_dict(const StateDict &state_dict, bool strict = true)
    {
        std::set<std::string> loaded;
        for (auto &kv : named_parameters())
        {
            auto it = state_dict.find(kv.first);
            if (it != state_dict.end())
            {
                if (kv.second->shape() != it->second.shape())
                    throw std::runtime_error("Shape mismatch for parameter '" + kv.first + "': expected " +
                                             kv.second->shape().to_string() + ", got " + it->second.shape().to_string());
                Tensor t              = it->second.clone();
                t.impl()->requires_grad = true;
                *kv.second            = Parameter(t);
                loaded.insert(kv.first);
            }
            else if (strict)
                throw std::runtime_error("Missing parameter '" + kv.first + "' in state_dict (strict mode)");
        }
        if (strict)
            for (auto &kv : state_dict)
                if (!loaded.count(kv.first))
                    throw std::runtime_error("Unexpected parameter '" + kv.first + "' in state_dict (strict mode)");
    }
    void load(const std::string &filepath, bool strict = true);  // origin::load + load_state_dict (module.cpp:214-218)
    // training / evaluation mode, propagated to the sub-modules (include/origin/nn/module.h:131-143)
    void train(bool mode = true)
    {
        training_ = mode;
        for (auto &kv : modules_)
            kv.second->train(mode);
    }
    void eval() { train(false); }
    bool is_training() const { return training_; }

  protected:
    void register_parameter(const std::string &name, Parameter &p) { params_.emplace_back(name, &p); }
    void register_module(const std::string &name, std::unique_ptr<Module> m) { modules_.emplace_back(name, std::move(m)); }
    std::vector<std::pair<std::string, Parameter *>> params_;
    std::vector<std::pair<std::string, std::unique_ptr<Module>>> modules_;
    bool training_ = true;
};

// weight {in, out} = randn * sqrt(1/in), bias {1, out} = 0 (src/nn/layers/linear.cpp:39-62).
class Linear : public Module
{
  public:
    Linear(int in_features, int out_features, bool bias = true, bool fused_relu = false)
        : in_(in_features), out_(out_features), use_bias_(bias), relu_(fused_relu)
    {
        if (in_features <= 0 || out_features <= 0)
            throw std::invalid_argument("Linear: in_features and out_features must be positive");
        Tensor w = Tensor::randn(Shape{(size_t)in_, (size_t)out_}, TensorOptions().requires_grad(true));
        Tensor ws = Tensor::empty(w.shape(), TensorOptions().requires_grad(true));
        odl_check(odl_scale(w.data_ptr<float>(), std::sqrt(1.0f / (float)in_), ws.data_ptr<float>(),
                            detail::i64(w.elements()), nullptr));
        weight_ = Parameter(ws);
        register_parameter("weight", weight_);
        if (use_bias_)
        {
            bias_ = Parameter(Tensor::zeros(Shape{1, (size_t)out_}, TensorOptions().requires_grad(true)));
            register_parameter("bias", bias_);
        }
    }
    Tensor forward(const Tensor &x) override
    {
        if (weight_.elements() == 0)
            throw std::runtime_error("Weight is empty in forward! weight_.shape() = " + weight_.shape().to_string());
        auto op = std::make_shared<functional::LinearOp>(in_, out_, use_bias_, ODL_W_IN_OUT, relu_);
        return use_bias_ ? op->call1({x, weight_, bias_}) : op->call1({x, weight_});
    }
    Parameter *weight() { return &weight_; }
    Parameter *bias() { return use_bias_ ? &bias_ : nullptr; }

  private:
    int in_, out_;
    bool use_bias_, relu_;
    Parameter weight_, bias_;
};

// Linear -> ReLU -> ... -> Linear, parameters named layer_i.weight / layer_i.bias (src/nn/models/mlp.cpp:11-61).
// gamma = 1, beta = 0 (parameters "weight", "bias"), running_mean = 0, running_var = 1; in training mode the running
// statistics follow running = momentum * running + (1 - momentum) * batch (src/nn/layers/batch_norm2d.cpp:12-83),
// applied by the statistics kernel itself instead of four device-to-host copies.  `act` fuses the ReLU / SiLU that
// follows the layer in the reference's CNN blocks.
class BatchNorm2d : public Module
{
  public:
    explicit BatchNorm2d(int num_features, float eps = 1e-5f, float momentum = 0.1f, int act = ODL_ACT_NONE)
        : num_features_(num_features), eps_(eps), momentum_(momentum), act_(act)
    {
        if (num_features <= 0)
            throw std::invalid_argument("BatchNorm2d: num_features must be positive, but got " + std::to_string(num_features));
        const Shape s{(size_t)num_features};
        gamma_        = Parameter(Tensor::ones(s, TensorOptions().requires_grad(true)));
        beta_         = Parameter(Tensor::zeros(s, TensorOptions().requires_grad(true)));
        running_mean_ = Tensor::zeros(s);
        running_var_  = Tensor::ones(s);
        register_parameter("weight", gamma_);
        register_parameter("bias", beta_);
    }
    Tensor forward(const Tensor &input) override
    {
        if (input.ndim() != 4)
            throw std::runtime_error("BatchNorm2d forward: input must be 4D (N, C, H, W), but got shape " +
                                     input.shape().to_string());
        if (input.shape()[1] != (size_t)num_features_)
            throw std::runtime_error("BatchNorm2d forward: input feature size " + std::to_string(input.shape()[1]) +
                                     " does not match num_features " + std::to_string(num_features_));
        auto op = std::make_shared<functional::BatchNorm>(is_training(), eps_, momentum_, 4, act_, is_training());
        return op->call1({input, gamma_, beta_, running_mean_, running_var_});
    }
    Parameter *weight() { return &gamma_; }
    Parameter *bias() { return &beta_; }
    const Tensor &running_mean() const { return running_mean_; }
    const Tensor &running_var() const { return running_var_; }

  private:
    int num_features_;
    float eps_, momentum_;
    int act_;
    Parameter gamma_, beta_;
    Tensor running_mean_, running_var_;
};

class MLP : public Module
{
  public:
    explicit MLP(const std::vector<int> &sizes)
    {
        if (sizes.size() < 2)
            throw std::invalid_argument("MLP requires at least 2 layer sizes (input and output), but got " +
                                        std::to_string(sizes.size()));
        for (size_t i = 0; i + 1 < sizes.size(); ++i)
        {
            auto l = std::make_unique<Linear>(sizes[i], sizes[i + 1], true, /*fused_relu=*/i + 2 < sizes.size());
            layers_.push_back(l.get());
            register_module("layer_" + std::to_string(i), std::move(l));
        }
    }
    Tensor forward(const Tensor &input) override
    {
        Tensor x = input;
        for (Linear *l : layers_)
            x = l->forward(x);
        return x;
    }

  private:
    std::vector<Linear *> layers_;
};

// weight {out, in, kh, kw} = randn * sqrt(2 / (in * kh * kw)), bias {out} = 0 (src/nn/layers/conv2d.cpp:15-109).  The
// kernels take one stride and one padding for both image axes: unequal pairs are refused.
class Conv2d : public Module
{
  public:
    Conv2d(int in_channels, int out_channels, std::pair<int, int> kernel_size, std::pair<int, int> stride = {1, 1},
           std::pair<int, int> pad = {0, 0}, bool bias = true)
        : stride_(stride.first), pad_(pad.first), use_bias_(bias)
    {
        if (in_channels <= 0)
            throw std::invalid_argument("Conv2d: in_channels must be positive, but got " + std::to_string(in_channels));
        if (out_channels <= 0)
            throw std::invalid_argument("Conv2d: out_channels must be positive, but got " + std::to_string(out_channels));
        if (kernel_size.first <= 0 || kernel_size.second <= 0)
            throw std::invalid_argument("Conv2d: kernel_size must be positive");
        if (stride.first <= 0 || stride.second <= 0)
            throw std::invalid_argument("Conv2d: stride must be positive");
        if (pad.first < 0 || pad.second < 0)
            throw std::invalid_argument("Conv2d: pad must be non-negative");
        if (stride.first != stride.second || pad.first != pad.second)
            throw std::invalid_argument("Conv2d: stride and pad must be the same for both image axes");
        const Shape ws{(size_t)out_channels, (size_t)in_channels, (size_t)kernel_size.first, (size_t)kernel_size.second};
        Tensor w  = Tensor::randn(ws, TensorOptions().requires_grad(true));
        Tensor sc = Tensor::empty(ws, TensorOptions().requires_grad(true));
        const float std_dev = std::sqrt(2.0f / (float)(in_channels * kernel_size.first * kernel_size.second));
        odl_check(odl_scale(w.data_ptr<float>(), std_dev, sc.data_ptr<float>(), detail::i64(w.elements()), nullptr));
        weight_ = Parameter(sc);
        register_parameter("weight", weight_);
        if (use_bias_)
        {
            bias_ = Parameter(Tensor::zeros(Shape{(size_t)out_channels}, TensorOptions().requires_grad(true)));
            register_parameter("bias", bias_);
        }
    }
    Conv2d(int in_channels, int out_channels, int kernel_size, int stride = 1, int pad = 0, bool bias = true)
        : Conv2d(in_channels, out_channels, {kernel_size, kernel_size}, {stride, stride}, {pad, pad}, bias)
    {
    }
    Tensor forward(const Tensor &input) override
    {
        return functional::conv2d(input, weight_, use_bias_ ? &bias_ : nullptr, stride_, pad_);
    }
    Parameter *weight() { return &weight_; }
    Parameter *bias() { return use_bias_ ? &bias_ : nullptr; }

  private:
    int stride_, pad_;
    bool use_bias_;
    Parameter weight_, bias_;
};

// BatchNorm over {N, C} inputs (src/nn/layers/batch_norm1d.cpp): the same kernels with one value per channel and sample.
class BatchNorm1d : public Module
{
  public:
    explicit BatchNorm1d(int num_features, float eps = 1e-5f, float momentum = 0.1f, int act = ODL_ACT_NONE)
        : num_features_(num_features), eps_(eps), momentum_(momentum), act_(act)
    {
        if (num_features <= 0)
            throw std::invalid_argument("BatchNorm1d: num_features must be positive, but got " + std::to_string(num_features));
        const Shape s{(size_t)num_features};
        gamma_        = Parameter(Tensor::ones(s, TensorOptions().requires_grad(true)));
        beta_         = Parameter(Tensor::zeros(s, TensorOptions().requires_grad(true)));
        running_mean_ = Tensor::zeros(s);
        running_var_  = Tensor::ones(s);
        register_parameter("weight", gamma_);
        register_parameter("bias", beta_);
    }
    Tensor forward(const Tensor &input) override
    {
        if (input.ndim() != 2 || input.shape()[1] != (size_t)num_features_)
            throw std::runtime_error("BatchNorm1d forward: input must be (N, " + std::to_string(num_features_) +
                                     "), but got shape " + input.shape().to_string());
        auto op = std::make_shared<functional::BatchNorm>(is_training(), eps_, momentum_, 2, act_, is_training());
        return op->call1({input, gamma_, beta_, running_mean_, running_var_});
    }
    const Tensor &running_mean() const { return running_mean_; }
    const Tensor &running_var() const { return running_var_; }

  private:
    int num_features_;
    float eps_, momentum_;
    int act_;
    Parameter gamma_, beta_;
    Tensor running_mean_, running_var_;
};

// Parameter-free layers (src/nn/layers/relu.cpp, flatten.cpp).
class ReLU : public Module
{
  public:
    Tensor forward(const Tensor &input) override { return functional::relu(input); }
};
class SiLU : public Module
{
  public:
    Tensor forward(const Tensor &input) override { return functional::silu(input); }
};
class Flatten : public Module
{
  public:
    explicit Flatten(int start_dim = 1, int end_dim = -1) : start_dim_(start_dim), end_dim_(end_dim) {}
    Tensor forward(const Tensor &input) override { return functional::flatten(input, start_dim_, end_dim_); }

  private:
    int start_dim_, end_dim_;
};

}  // namespace nn

// Modules applied one after the other (include/origin/nn/sequential.h, src/nn/sequential.cpp:7-62): add(), forward(),
// parameters(), operator[], size() as in the reference.  One deliberate difference: the reference keeps the children in
// a private vector that Module::named_parameters() never sees, so its state_dict() of a Sequential is empty; here the
// children are registered under "0", "1", ... and state_dict() / load_state_dict() / checkpoints cover them.
class Sequential : public nn::Module
{
  public:
    void add(std::unique_ptr<nn::Module> module)
    {
        if (!module)
            throw std::invalid_argument("Sequential::add: null module");
        order_.push_back(module.get());
        register_module(std::to_string(order_.size() - 1), std::move(module));
    }
    Tensor forward(const Tensor &input) override
    {
        Tensor out = input;
        for (nn::Module *m : order_)
            out = m->forward(out);
        return out;
    }
    nn::Module &operator[](size_t index)
    {
        if (index >= order_.size())
            throw std::runtime_error("Index " + std::to_string(index) + " out of range for Sequential with " +
                                     std::to_string(order_.size()) + " modules");
        return *order_[index];
    }
    size_t size() const { return order_.size(); }

  private:
    std::vector<nn::Module *> order_;
};

// ------------------------------------------------------------------------------------------------ optimizers
class Optimizer
{
  public:
    using State = std::unordered_map<std::string, std::any>;
    explicit Optimizer(nn::Module &target) : target_(&target), params_(target.parameters()) {}
    virtual ~Optimizer() = default;
    // Configuration scalars (float / bool), per-parameter buffers as a StateDict and, for Adam, the step counts
    // (include/origin/optim/optimizer.h:66-80).
    virtual State state_dict() = 0;
    virtual void load_state_dict(const State &state) = 0;
    void register_hook(std::function<void(std::vector<Parameter *> &)> h) { hooks_.push_back(std::move(h)); }
    void zero_grad()
    {
        for (Parameter *p : params_)
            p->clear_grad();
    }
    // hooks first, then step_one per parameter that has a gradient (src/optim/optimizer.cpp:19-53)
    void step()
    {
        std::vector<Parameter *> with_grad;
        for (Parameter *p : params_)
            if (p->has_grad())
                with_grad.push_back(p);
        for (auto &h : hooks_)
            h(with_grad);
        for (Parameter *p : with_grad)
            step_one(*p);
    }

  protected:
    virtual void step_one(Parameter &p) = 0;
    // buffers of `by_param` under "<prefix><parameter name>", the way the reference names them (adam.cpp:126-147)
    template <typename Map, typename Get>
    nn::Module::StateDict named_buffers(const Map &by_param, const std::string &prefix, Get get)
    {
        nn::Module::StateDict out;
        for (auto &kv : target_->named_parameters())
        {
            auto it = by_param.find(kv.second);
            if (it != by_param.end())
                out[prefix + kv.first] = get(it->second);
        }
        return out;
    }
    template <typename T>
    static bool fetch(const State &s, const char *key, T &out)
    {
        auto it = s.find(key);
        if (it == s.end())
            return false;
        out = std::any_cast<T>(it->second);
        return true;
    }
    nn::Module *target_;
    std::vector<Parameter *> params_;
    std::vector<std::function<void(std::vector<Parameter *> &)>> hooks_;
};

// grad += rate * param, in place on the gradient tensor (include/origin/optim/hooks.h:21-68).
class WeightDecay
{
  public:
    explicit WeightDecay(float rate = 1e-4f) : rate_(rate) {}
    std::function<void(std::vector<Parameter *> &)> hook()
    {
        const float rate = rate_;
        return [rate](std::vector<Parameter *> &params) {
            for (Parameter *p : params)
                if (p && p->has_grad())
                    odl_check(odl_axpy(rate, p->data_ptr<float>(), p->grad().data_ptr<float>(), (int64_t)p->elements(),
                                       nullptr));
        };
    }

  private:
    float rate_;
};

class SGD : public Optimizer  // src/optim/sgd.cpp:18-75, one fused in-place kernel per parameter
{
  public:
    SGD(nn::Module &target, float lr, float momentum = 0.0f, float weight_decay = 0.0f, bool nesterov = false)
        : Optimizer(target), lr_(lr), momentum_(momentum), wd_(weight_decay), nesterov_(nesterov)
    {
    }
    // lr, momentum, weight_decay, nesterov and "momentum_buffers" {momentum_<param>} (src/optim/sgd.cpp:77-115)
    State state_dict() override
    {
        State st;
        st["lr"]               = lr_;
        st["momentum"]         = momentum_;
        st["weight_decay"]     = wd_;
        st["nesterov"]         = nesterov_;
        st["momentum_buffers"] = named_buffers(buf_, "momentum_", [](const Tensor &t) { return t; });
        return st;
    }
    void load_state_dict(const State &st) override
    {
        fetch(st, "lr", lr_);
        fetch(st, "momentum", momentum_);
        fetch(st, "weight_decay", wd_);
        fetch(st, "nesterov", nesterov_);
        nn::Module::StateDict bufs;
        if (fetch(st, "momentum_buffers", bufs))
        {
            buf_.clear();
            auto named = target_->named_parameters();
            for (auto &kv : bufs)
                if (kv.first.rfind("momentum_", 0) == 0 && named.count(kv.first.substr(9)))
                    buf_[named[kv.first.substr(9)]] = kv.second.clone();
        }
    }

  protected:
    void step_one(Parameter &p) override
    {
        float *buf = nullptr;
        if (momentum_ > 0.0f)
        {
            auto it = buf_.find(&p);
            if (it == buf_.end())
                it = buf_.emplace(&p, Tensor::zeros(p.shape())).first;
            buf = it->second.data_ptr<float>();
        }
        odl_check(odl_sgd_step(p.data_ptr<float>(), p.grad().data_ptr<float>(), buf, nullptr, (int64_t)p.elements(), lr_,
                               momentum_, wd_, nesterov_ ? 1 : 0, 0.0f, 1.0f, nullptr));
    }

  private:
    float lr_, momentum_, wd_;
    bool nesterov_;
    std::unordered_map<Parameter *, Tensor> buf_;
};

class Adam : public Optimizer  // src/optim/adam.cpp:19-114
{
  public:
    Adam(nn::Module &target, float lr = 1e-3f, float beta1 = 0.9f, float beta2 = 0.999f, float eps = 1e-8f)
        : Optimizer(target), lr_(lr), b1_(beta1), b2_(beta2), eps_(eps)
    {
    }
    // lr, beta1, beta2, eps, "m_buffers" {m_<param>}, "v_buffers" {v_<param>}, "step_counts" {step_<param>}
    // (src/optim/adam.cpp:116-193)
    State state_dict() override
    {
        State st;
        st["lr"]        = lr_;
        st["beta1"]     = b1_;
        st["beta2"]     = b2_;
        st["eps"]       = eps_;
        st["m_buffers"] = named_buffers(state_, "m_", [](const PerParam &s) { return s.m; });
        st["v_buffers"] = named_buffers(state_, "v_", [](const PerParam &s) { return s.v; });
        std::unordered_map<std::string, int> steps;
        for (auto &kv : target_->named_parameters())
        {
            auto it = state_.find(kv.second);
            if (it != state_.end())
                steps["step_" + kv.first] = it->second.t;
        }
        st["step_counts"] = steps;
        return st;
    }
    void load_state_dict(const State &st) override  // src/optim/adam.cpp:195-277
    {
        fetch(st, "lr", lr_);
        fetch(st, "beta1", b1_);
        fetch(st, "beta2", b2_);
        fetch(st, "eps", eps_);
        auto named = target_->named_parameters();
        nn::Module::StateDict m, v;
        std::unordered_map<std::string, int> steps;
        const bool has_m = fetch(st, "m_buffers", m), has_v = fetch(st, "v_buffers", v);
        const bool has_t = fetch(st, "step_counts", steps);
        if (has_m || has_v || has_t)
            state_.clear();
        auto slot = [&](const std::string &key, size_t prefix) -> PerParam * {
            auto it = named.find(key.substr(prefix));
            if (it == named.end())
                return nullptr;
            auto ins = state_.find(it->second);
            if (ins == state_.end())
                ins = state_.emplace(it->second, PerParam{Tensor::zeros(it->second->shape()),
                                                          Tensor::zeros(it->second->shape()), 0}).first;
            return &ins->second;
        };
        for (auto &kv : m)
            if (kv.first.rfind("m_", 0) == 0)
                if (PerParam *s = slot(kv.first, 2))
                    s->m = kv.second.clone();
        for (auto &kv : v)
            if (kv.first.rfind("v_", 0) == 0)
                if (PerParam *s = slot(kv.first, 2))
                    s->v = kv.second.clone();
        for (auto &kv : steps)
            if (kv.first.rfind("step_", 0) == 0)
                if (PerParam *s = slot(kv.first, 5))
                    s->t = kv.second;
    }

  protected:
    void step_one(Parameter &p) override
    {
        auto it = state_.find(&p);
        if (it == state_.end())
            it = state_.emplace(&p, PerParam{Tensor::zeros(p.shape()), Tensor::zeros(p.shape()), 0}).first;
        PerParam &s = it->second;
        s.t += 1;
        odl_check(odl_adam_step(p.data_ptr<float>(), p.grad().data_ptr<float>(), s.m.data_ptr<float>(),
                                s.v.data_ptr<float>(), nullptr, (int64_t)p.elements(), s.t, lr_, b1_, b2_, eps_, 0.0f, 1.0f,
                                nullptr));
    }

  private:
    struct PerParam
    {
        Tensor m, v;
        int t;
    };
    float lr_, b1_, b2_, eps_;
    std::unordered_map<Parameter *, PerParam> state_;
};

// ------------------------------------------------------------------------------------------------ .odl files, checkpoints
// State-dict files in the reference's format (src/io/model_io.cpp:114-273), little endian, size_t = 8 bytes:
//   u32 magic 0x4F444C00 | u32 version 1 | u64 count | per tensor: u64 name length, name | u64 rank, u64 dims[rank] |
//   i32 dtype (reference enum: 0 float32, 3 int32) | i32 device type (1 = CUDA), i32 device index | raw values.
// Tensors of this layer are float32 or int32/int64; like the reference, save() rejects what it cannot represent
// (int64), and load() rejects float64 records, which have no tensor type here.
using StateDict = nn::Module::StateDict;

namespace detail
{
template <typename T>
inline void put(std::ofstream &out, const T &v)
{
    out.write(reinterpret_cast<const char *>(&v), sizeof(T));
}
template <typename T>
inline T get(std::ifstream &in, const char *what)
{
    T v;
    in.read(reinterpret_cast<char *>(&v), sizeof(T));
    if (in.fail())
        throw std::runtime_error(std::string("Failed to read ") + what + " from file");
    return v;
}
inline std::string checkpoint_dir(const std::string &filepath)
{
    return filepath.size() > 5 && filepath.substr(filepath.size() - 5) == ".ckpt" ? filepath.substr(0, filepath.size() - 5)
                                                                                    : filepath;
}
}  // namespace detail

inline void save(const StateDict &state_dict, const std::string &filepath)
{
    std::ofstream out(filepath, std::ios::binary);
    if (!out.is_open())
        throw std::runtime_error("Failed to open file for writing: " + filepath);
    int device = 0;
    cudaGetDevice(&device);
    detail::put<uint32_t>(out, 0x4F444C00u);
    detail::put<uint32_t>(out, 1u);
    detail::put<uint64_t>(out, state_dict.size());
    std::vector<std::string> names;
    for (auto &kv : state_dict)
        names.push_back(kv.first);
    std::sort(names.begin(), names.end());  // the reference writes hash-map order; the order carries no meaning
    for (const std::string &name : names)
    {
        const Tensor &t = state_dict.at(name);
        detail::put<uint64_t>(out, name.size());
        out.write(name.data(), (std::streamsize)name.size());
        detail::put<uint64_t>(out, t.shape().size());
        for (size_t d : t.shape().dims())
            detail::put<uint64_t>(out, d);
        if (t.dtype() != DataType::kFloat32 && t.dtype() != DataType::kInt32)
            throw std::runtime_error("Unsupported dtype for saving: " + std::to_string(t.dtype() == DataType::kInt64 ? 4 : -1));
        detail::put<int32_t>(out, t.dtype() == DataType::kFloat32 ? 0 : 3);
        detail::put<int32_t>(out, 1);
        detail::put<int32_t>(out, device);
        if (t.dtype() == DataType::kFloat32)
        {
            auto v = t.to_vector<float>();
            out.write(reinterpret_cast<const char *>(v.data()), (std::streamsize)(v.size() * sizeof(float)));
        }
        else
        {
            auto v = t.to_vector<int32_t>();
            out.write(reinterpret_cast<const char *>(v.data()), (std::streamsize)(v.size() * sizeof(int32_t)));
        }
    }
    out.close();
    if (out.fail())
        throw std::runtime_error("Failed to write to file: " + filepath);
}

inline StateDict load(const std::string &filepath)
{
    std::ifstream in(filepath, std::ios::binary);
    if (!in.is_open())
        throw std::runtime_error("Failed to open file for reading: " + filepath);
    uint32_t magic = 0;
    in.read(reinterpret_cast<char *>(&magic), sizeof(magic));
    if (in.fail() || magic != 0x4F444C00u)
        throw std::runtime_error("Invalid file format or corrupted file: " + filepath);
    uint32_t version = 0;
    in.read(reinterpret_cast<char *>(&version), sizeof(version));
    if (in.fail() || version != 1)
        throw std::runtime_error("Unsupported file version: " + std::to_string(version));
    const uint64_t count = detail::get<uint64_t>(in, "parameter count");
    StateDict sd;
    for (uint64_t i = 0; i < count; ++i)
    {
        const uint64_t len = detail::get<uint64_t>(in, "string length");
        std::string name(len, '\0');
        in.read(&name[0], (std::streamsize)len);
        if (in.fail())
            throw std::runtime_error("Failed to read string data from file");
        const uint64_t rank = detail::get<uint64_t>(in, "shape dimensions");
        std::vector<size_t> dims(rank);
        for (uint64_t d = 0; d < rank; ++d)
            dims[d] = detail::get<uint64_t>(in, "shape dimension");
        const int32_t code = detail::get<int32_t>(in, "dtype");
        detail::get<int32_t>(in, "device");
        detail::get<int32_t>(in, "device");  // tensors of this layer always live on the current CUDA device
        Shape shape(dims);
        if (code == 0)
        {
            std::vector<float> v(shape.elements());
            in.read(reinterpret_cast<char *>(v.data()), (std::streamsize)(v.size() * sizeof(float)));
            if (in.fail())
                throw std::runtime_error("Failed to read tensor data for parameter '" + name + "'");
            sd[name] = Tensor(v, shape);
        }
        else if (code == 3)
        {
            std::vector<int32_t> v(shape.elements());
            in.read(reinterpret_cast<char *>(v.data()), (std::streamsize)(v.size() * sizeof(int32_t)));
            if (in.fail())
                throw std::runtime_error("Failed to read tensor data for parameter '" + name + "'");
            sd[name] = Tensor(v, shape);
        }
        else
            throw std::runtime_error("Unsupported dtype for loading: " + std::to_string(code));
    }
    return sd;
}

inline void nn::Module::load(const std::string &filepath, bool strict)
{
    load_state_dict(origin::load(filepath), strict);
}

// include/origin/io/checkpoint.h:13-25.  A checkpoint is a DIRECTORY (the path minus a trailing ".ckpt") with model.odl
// and metadata.json written exactly as the reference writes them (src/io/checkpoint.cpp:15-75), plus optimizer.odl,
// which the reference names and never writes: here it holds every StateDict found in optimizer_state_dict (the
// m_/v_/momentum_ buffers) and the Adam step counts as int32 tensors of shape {1}, so that training resumes on the
// same trajectory.  The reference's loader ignores the extra file.
struct Checkpoint
{
    StateDict model_state_dict;
    std::unordered_map<std::string, Optimizer::State> optimizer_state_dict;
    int epoch  = -1;
    int step   = -1;
    float loss = 0.0f;
    std::string optimizer_type;
    std::unordered_map<std::string, float> optimizer_config;
};

inline void save(const Checkpoint &checkpoint, const std::string &filepath)
{
    namespace fs = std::filesystem;
    const std::string dir = detail::checkpoint_dir(filepath);
    try
    {
        fs::create_directories(dir);
    }
    catch (const std::exception &e)
    {
        throw std::runtime_error("Failed to create checkpoint directory '" + dir + "': " + e.what());
    }
    save(checkpoint.model_state_dict, dir + "/model.odl");
    StateDict opt;
    for (auto &named : checkpoint.optimizer_state_dict)
        for (auto &kv : named.second)
        {
            if (kv.second.type() == typeid(StateDict))
                for (auto &t : std::any_cast<const StateDict &>(kv.second))
                    opt[t.first] = t.second;
            else if (kv.second.type() == typeid(std::unordered_map<std::string, int>))
                for (auto &t : std::any_cast<const std::unordered_map<std::string, int> &>(kv.second))
                    opt[t.first] = Tensor(std::vector<int32_t>{t.second}, Shape{1});
        }
    if (!opt.empty())
        save(opt, dir + "/optimizer.odl");
    std::ofstream meta(dir + "/metadata.json");
    if (!meta.is_open())
        throw std::runtime_error("Failed to open metadata file for writing: " + dir + "/metadata.json");
    meta << "{\n";
    meta << "  \"format_version\": \"1.0\",\n";
    meta << "  \"format_type\": \"origindl_checkpoint\",\n";
    meta << "  \"epoch\": " << checkpoint.epoch << ",\n";
    meta << "  \"step\": " << checkpoint.step << ",\n";
    meta << "  \"loss\": " << checkpoint.loss << ",\n";
    meta << "  \"optimizer_type\": \"" << checkpoint.optimizer_type << "\",\n";
    meta << "  \"optimizer_config\": {\n";
    bool first = true;
    for (auto &kv : checkpoint.optimizer_config)
    {
        if (!first)
            meta << ",\n";
        meta << "    \"" << kv.first << "\": " << kv.second;
        first = false;
    }
    meta << "\n  }\n";
    meta << "}\n";
}

// src/io/checkpoint.cpp:77-226, including its line-oriented metadata parser.  When optimizer.odl exists its tensors
// come back under optimizer_state_dict[<optimizer_type in lower case>] in the shape Optimizer::load_state_dict takes.
inline Checkpoint load_checkpoint(const std::string &filepath)
{
    namespace fs = std::filesystem;
    const std::string dir = detail::checkpoint_dir(filepath);
    if (!fs::exists(dir) || !fs::is_directory(dir))
        throw std::runtime_error("Checkpoint directory does not exist: " + dir);
    Checkpoint ck;
    if (!fs::exists(dir + "/model.odl"))
        throw std::runtime_error("Model file not found in checkpoint: " + dir + "/model.odl");
    ck.model_state_dict = load(dir + "/model.odl");
    if (!fs::exists(dir + "/metadata.json"))
        throw std::runtime_error("Metadata file not found in checkpoint: " + dir + "/metadata.json");
    std::ifstream meta(dir + "/metadata.json");
    if (!meta.is_open())
        throw std::runtime_error("Failed to open metadata file: " + dir + "/metadata.json");
    auto value_of = [](const std::string &line) {
        std::string v = line.substr(line.find(':') + 1);
        v.erase(0, v.find_first_not_of(" \t,"));
        v.erase(v.find_last_not_of(" \t,") + 1);
        return v;
    };
    std::string line;
    while (std::getline(meta, line))
    {
        if (line.find(':') == std::string::npos)
            continue;
        if (line.find("\"epoch\"") != std::string::npos)
            ck.epoch = std::atoi(value_of(line).c_str());
        if (line.find("\"step\"") != std::string::npos)
            ck.step = std::atoi(value_of(line).c_str());
        if (line.find("\"loss\"") != std::string::npos)
            ck.loss = (float)std::atof(value_of(line).c_str());
        if (line.find("\"optimizer_type\"") != std::string::npos)
        {
            const std::string v = line.substr(line.find(':') + 1);
            const size_t a = v.find('"'), b = v.find('"', a + 1);
            if (a != std::string::npos && b != std::string::npos)
                ck.optimizer_type = v.substr(a + 1, b - a - 1);
        }
        for (const char *key : {"lr", "beta1", "beta2", "eps"})
            if (line.find(std::string("\"") + key + "\"") != std::string::npos)
                ck.optimizer_config[key] = (float)std::atof(value_of(line).c_str());
    }
    if (fs::exists(dir + "/optimizer.odl"))
    {
        StateDict m, v, mom;
        std::unordered_map<std::string, int> steps;
        for (auto &kv : load(dir + "/optimizer.odl"))
        {
            if (kv.first.rfind("m_", 0) == 0 && kv.first.rfind("momentum_", 0) != 0)
                m[kv.first] = kv.second;
            else if (kv.first.rfind("v_", 0) == 0)
                v[kv.first] = kv.second;
            else if (kv.first.rfind("momentum_", 0) == 0)
                mom[kv.first] = kv.second;
            else if (kv.first.rfind("step_", 0) == 0)
                steps[kv.first] = kv.second.to_vector<int32_t>()[0];
        }
        std::string key = ck.optimizer_type;
        std::transform(key.begin(), key.end(), key.begin(), [](unsigned char c) { return (char)std::tolower(c); });
        Optimizer::State st;
        for (auto &kv : ck.optimizer_config)
            st[kv.first] = kv.second;
        if (!m.empty())
            st["m_buffers"] = m;
        if (!v.empty())
            st["v_buffers"] = v;
        if (!mom.empty())
            st["momentum_buffers"] = mom;
        if (!steps.empty())
            st["step_counts"] = steps;
        ck.optimizer_state_dict[key] = st;
    }
    return ck;
}

// ------------------------------------------------------------------------------------------------------------------
// Dataset / DataLoader (include/origin/data/dataset.h:12-26, include/origin/data/dataloader.h:14-52,
// src/data/dataloader.cpp:11-146).  Same interface, batch order and error behaviour: samples are flattened to
// {batch, elements}; integer labels come out as int64, other labels as float32; the last batch of an epoch is short;
// next() past the end throws std::runtime_error.  What differs is where the work happens: the reference calls get_item()
// for every sample of every batch and assembles the batch on the host.  Here the data set is read ONCE (get_item() for
// every index at the first next(), device-to-device copies into one resident matrix) and every batch is one row-gather
// kernel (odl_gather_rows) driven by the epoch's index list, which is uploaded at reset().  A data set whose get_item() is
// not a pure function of the index (augmentation) must pass cache = false; batches are then gathered from fresh
// get_item() calls as in the reference.  The reference seeds its shuffle from std::random_device; `seed` makes the order
// reproducible (0 = from std::random_device).
class Dataset
{
  public:
    virtual ~Dataset() = default;
    virtual std::pair<Tensor, Tensor> get_item(size_t index) = 0;
    virtual size_t size() const = 0;
    bool valid_index(size_t index) const { return index < size(); }
};

class DataLoader
{
  public:
    DataLoader(Dataset &dataset, size_t batch_size = 1, bool shuffle = false, uint64_t seed = 0, bool cache = true)
        : dataset_(&dataset), batch_size_(batch_size), shuffle_(shuffle), cache_(cache),
          gen_(seed ? seed : std::random_device{}())
    {
        if (batch_size_ == 0)
            throw std::invalid_argument("DataLoader: batch size must be positive");
        reset_indices();
    }

    bool has_next() const { return current_index_ < indices_.size(); }
    size_t dataset_size() const { return dataset_->size(); }
    size_t batch_size() const { return batch_size_; }
    void reset() { reset_indices(); }

    std::pair<Tensor, Tensor> next()
    {
        if (!has_next())
            throw std::runtime_error(
                "DataLoader::next() called when no more data available. Use has_next() to check before calling next().");
        const size_t rows = std::min(batch_size_, indices_.size() - current_index_);
        if (!cache_)
        {
            // gather this batch's samples from fresh get_item() calls, then the same device-side assembly
            std::vector<size_t> ids(indices_.begin() + current_index_, indices_.begin() + current_index_ + rows);
            Resident batch = read(ids);
            current_index_ += rows;
            return {batch.x, batch.t};
        }
        if (!all_.x.defined())
        {
            std::vector<size_t> ids(dataset_->size());
            for (size_t i = 0; i < ids.size(); ++i)
                ids[i] = i;
            all_ = read(ids);
        }
        if (!dev_indices_.defined())
        {
            std::vector<int64_t> idx(indices_.begin(), indices_.end());
            dev_indices_ = Tensor(idx, Shape{idx.size()}, dtype(DataType::kInt64));
        }
        const int64_t cols = static_cast<int64_t>(all_.x.shape()[1]), n = static_cast<int64_t>(all_.x.shape()[0]);
        Tensor x = Tensor::empty(Shape{rows, static_cast<size_t>(cols)});
        const int64_t *idx = dev_indices_.data_ptr<int64_t>() + current_index_;
        Tensor t;
        if (all_.t.dtype() == DataType::kInt64)
        {
            t = Tensor::empty(Shape{rows}, dtype(DataType::kInt64));
            odl_check(odl_gather_rows(all_.x.data_ptr<float>(), cols, n, idx, static_cast<int64_t>(rows), cols, x.data_ptr<float>(),
                                      cols, all_.t.data_ptr<int64_t>(), t.data_ptr<int64_t>(), nullptr));
        }
        else
        {
            t = Tensor::empty(Shape{rows});
            odl_check(odl_gather_rows(all_.x.data_ptr<float>(), cols, n, idx, static_cast<int64_t>(rows), cols, x.data_ptr<float>(),
                                      cols, nullptr, nullptr, nullptr));
            odl_check(odl_gather_rows(all_.t.data_ptr<float>(), 1, n, idx, static_cast<int64_t>(rows), 1, t.data_ptr<float>(), 1,
                                      nullptr, nullptr, nullptr));
        }
        current_index_ += rows;
        return {x, t};
    }

  private:
    struct Resident
    {
        Tensor x;  // {samples, elements} float32
        Tensor t;  // {samples} int64 (integer labels) or float32
    };

    // Samples ids[0..] as one device matrix and one label vector (DataLoader::next's per-sample loop, done with
    // device-to-device copies; integer labels of any width become int64 as in the reference).
    Resident read(const std::vector<size_t> &ids)
    {
        Resident r;
        if (ids.empty())
            return r;
        auto first            = dataset_->get_item(ids[0]);
        const size_t elements = first.first.elements();
        const DataType ldt    = first.second.dtype();
        const bool int_labels = ldt != DataType::kFloat32;
        r.x                   = Tensor::empty(Shape{ids.size(), elements});
        Tensor raw = Tensor::empty(Shape{ids.size()}, dtype(ldt));  // labels in the data set's own type
        for (size_t i = 0; i < ids.size(); ++i)
        {
            auto item = i == 0 ? first : dataset_->get_item(ids[i]);
            if (item.first.elements() != elements)
                throw std::runtime_error("Inconsistent input shapes in dataset: expected " + std::to_string(elements) +
                                         " elements, got " + std::to_string(item.first.elements()));
            if (item.first.dtype() != DataType::kFloat32 || item.second.dtype() != ldt || item.second.elements() != 1)
                throw std::runtime_error("DataLoader: inputs must be float32 and labels single values of one type");
            cuda_check(cudaMemcpyAsync(r.x.data_ptr<float>() + i * elements, item.first.data_ptr<float>(), elements * 4,
                                       cudaMemcpyDeviceToDevice, nullptr),
                       "DataLoader: sample copy");
            cuda_check(cudaMemcpyAsync(static_cast<char *>(raw.data_ptr<void>()) + i * element_size(ldt),
                                       item.second.data_ptr<void>(), element_size(ldt), cudaMemcpyDeviceToDevice, nullptr),
                       "DataLoader: label copy");
        }
        if (!int_labels || ldt == DataType::kInt64)
        {
            r.t = raw;
        }
        else
        {
            std::vector<int32_t> narrow = raw.to_vector<int32_t>();
            std::vector<int64_t> wide(narrow.begin(), narrow.end());
            r.t = Tensor(wide, Shape{wide.size()}, dtype(DataType::kInt64));
        }
        synchronize();  // the items' storage may be released once this returns
        return r;
    }

    void reset_indices()
    {
        indices_.resize(dataset_->size());
        for (size_t i = 0; i < indices_.size(); ++i)
            indices_[i] = i;
        if (shuffle_)
            std::shuffle(indices_.begin(), indices_.end(), gen_);
        current_index_ = 0;
        dev_indices_   = Tensor();
    }

    Dataset *dataset_;
    size_t batch_size_;
    bool shuffle_, cache_;
    std::mt19937_64 gen_;
    std::vector<size_t> indices_;
    size_t current_index_ = 0;
    Resident all_;
    Tensor dev_indices_;
};

}  // namespace origin

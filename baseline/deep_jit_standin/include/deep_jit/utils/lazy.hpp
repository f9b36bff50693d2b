// Stand-in for third-party/deep_jit of the reference: an object created on first use.
// Interface read off the call sites (csrc/runtime/jit.hpp:12,22, csrc/runtime/runtime.hpp:104, csrc/apis/config.hpp:12-14):
// constructible from nullptr (nothing to create: using it is an error) or from a factory returning shared_ptr<T>;
// operator-> creates the object on first use; assigning a new LazyInit drops the old object.
#pragma once

#include <functional>
#include <memory>
#include <mutex>
#include <stdexcept>

namespace deep_jit {

template <typename T>
class LazyInit {
public:
    using Factory = std::function<std::shared_ptr<T>()>;

    LazyInit(std::nullptr_t) {}                         // NOLINT: implicit on purpose
    LazyInit(Factory factory) : factory_(std::move(factory)) {}   // NOLINT

    LazyInit(const LazyInit& other) : factory_(other.factory_), object_(other.object_) {}
    LazyInit& operator=(const LazyInit& other) {
        if (this != &other) {
            std::lock_guard<std::mutex> lock(mutex_);
            factory_ = other.factory_;
            object_ = other.object_;
        }
        return *this;
    }

    T* operator->() { return get().get(); }
    T& operator*() { return *get(); }

    std::shared_ptr<T> get() {
        std::lock_guard<std::mutex> lock(mutex_);
        if (object_ == nullptr) {
            if (!factory_) throw std::runtime_error("deep_jit stand-in: object used before it was initialised (call init first)");
            object_ = factory_();
        }
        return object_;
    }

    bool created() const { return object_ != nullptr; }

private:
    Factory factory_;
    std::shared_ptr<T> object_;
    std::mutex mutex_;
};

}  // namespace deep_jit

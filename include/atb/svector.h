// Small vector used by VariantPack: up to 64 elements inline, at most 256 on the heap.
// Same contract as include/atb/svector.h of the reference (capacities :27-28, bounds-checked
// operator[]/at :192-241, MaxSizeExceeded on overflow); the implementation is independent.
#ifndef ATB_SVECTOR_H
#define ATB_SVECTOR_H
#include <cstddef>
#include <exception>
#include <initializer_list>
#include <new>
#include <ostream>
#include <stdexcept>

namespace atb {
constexpr std::size_t MAX_SVECTOR_SIZE = 256;
constexpr std::size_t DEFAULT_SVECTOR_SIZE = 64;

struct MaxSizeExceeded : public std::exception {};

template <class T> class SVector {
public:
    SVector() = default;
    SVector(std::initializer_list<T> list) { Assign(list.begin(), list.size()); }
    explicit SVector(std::size_t n, const T &value = T())
    {
        Grow(n);
        for (std::size_t i = 0; i < n; ++i) {
            Ptr()[i] = value;
        }
        size_ = n;
    }
    SVector(const SVector &other) { Assign(other.data(), other.size_); }
    SVector &operator=(const SVector &other)
    {
        if (this != &other) {
            Assign(other.data(), other.size_);
        }
        return *this;
    }
    SVector &operator=(std::initializer_list<T> list)
    {
        Assign(list.begin(), list.size());
        return *this;
    }
    ~SVector() { delete[] heap_; }

    void push_back(const T &v)
    {
        Grow(size_ + 1);
        Ptr()[size_++] = v;
    }
    void insert(std::size_t pos, const T &v)
    {
        if (pos > size_) {
            throw std::out_of_range("SVector insert position out of range");
        }
        Grow(size_ + 1);
        T *p = Ptr();
        for (std::size_t i = size_; i > pos; --i) {
            p[i] = p[i - 1];
        }
        p[pos] = v;
        ++size_;
    }
    void resize(std::size_t n)
    {
        Grow(n);
        size_ = n;
    }
    void reserve(std::size_t n) { Grow(n); }
    void clear() noexcept { size_ = 0; }
    bool empty() const noexcept { return size_ == 0; }
    std::size_t size() const noexcept { return size_; }

    T *data() noexcept { return Ptr(); }
    const T *data() const noexcept { return Ptr(); }
    T *begin() noexcept { return Ptr(); }
    const T *begin() const noexcept { return Ptr(); }
    T *end() noexcept { return Ptr() + size_; }
    const T *end() const noexcept { return Ptr() + size_; }

    T &at(std::size_t i)
    {
        if (i >= size_) {
            throw std::out_of_range("SVector index out of range");
        }
        return Ptr()[i];
    }
    const T &at(std::size_t i) const
    {
        if (i >= size_) {
            throw std::out_of_range("SVector index out of range");
        }
        return Ptr()[i];
    }
    T &operator[](std::size_t i) { return at(i); }
    const T &operator[](std::size_t i) const { return at(i); }

    bool operator==(const SVector &o) const
    {
        if (size_ != o.size_) {
            return false;
        }
        for (std::size_t i = 0; i < size_; ++i) {
            if (!(Ptr()[i] == o.Ptr()[i])) {
                return false;
            }
        }
        return true;
    }
    bool operator!=(const SVector &o) const { return !(*this == o); }
    bool operator<(const SVector &o) const
    {
        if (size_ != o.size_) {
            return size_ < o.size_;
        }
        for (std::size_t i = 0; i < size_; ++i) {
            if (Ptr()[i] != o.Ptr()[i]) {
                return Ptr()[i] < o.Ptr()[i];
            }
        }
        return false;
    }

private:
    T *Ptr() noexcept { return heap_ ? heap_ : inline_; }
    const T *Ptr() const noexcept { return heap_ ? heap_ : inline_; }
    void Grow(std::size_t n)
    {
        if (n > MAX_SVECTOR_SIZE) {
            throw MaxSizeExceeded();
        }
        if (n > DEFAULT_SVECTOR_SIZE && !heap_) {
            T *h = new T[MAX_SVECTOR_SIZE]();
            for (std::size_t i = 0; i < size_; ++i) {
                h[i] = inline_[i];
            }
            heap_ = h;
        }
    }
    void Assign(const T *src, std::size_t n)
    {
        size_ = 0;
        Grow(n);
        for (std::size_t i = 0; i < n; ++i) {
            Ptr()[i] = src[i];
        }
        size_ = n;
    }

    std::size_t size_ = 0;
    T inline_[DEFAULT_SVECTOR_SIZE] = {};
    T *heap_ = nullptr;
};

template <class T> std::ostream &operator<<(std::ostream &os, const SVector<T> &v)
{
    for (std::size_t i = 0; i < v.size(); ++i) {
        os << (i ? "," : "") << v.at(i);
    }
    return os;
}
} // namespace atb
#endif

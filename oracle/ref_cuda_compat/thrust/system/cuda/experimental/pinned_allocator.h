// Stand-in for the header Thrust no longer ships: a page-locked host allocator with the
// name the reference's sources use (io.h:6, builder.h:7, partition.cuh:7).  Only used to
// compile the reference as a checker / baseline; never part of the product.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <limits>
#include <new>

namespace thrust {
namespace cuda {
namespace experimental {

template <typename T>
class pinned_allocator {
 public:
  typedef T value_type;
  typedef T *pointer;
  typedef const T *const_pointer;
  typedef T &reference;
  typedef const T &const_reference;
  typedef std::size_t size_type;
  typedef std::ptrdiff_t difference_type;
  template <typename U>
  struct rebind {
    typedef pinned_allocator<U> other;
  };
  pinned_allocator() {}
  pinned_allocator(const pinned_allocator &) {}
  template <typename U>
  pinned_allocator(const pinned_allocator<U> &) {}
  pointer address(reference r) { return &r; }
  const_pointer address(const_reference r) { return &r; }
  pointer allocate(size_type n, const_pointer = 0) {
    if (n > max_size()) throw std::bad_alloc();
    void *p = nullptr;
    if (cudaMallocHost(&p, n * sizeof(T)) != cudaSuccess) {
      cudaGetLastError();
      throw std::bad_alloc();
    }
    return static_cast<pointer>(p);
  }
  void deallocate(pointer p, size_type) { cudaFreeHost(p); }
  size_type max_size() const { return (std::numeric_limits<size_type>::max)() / sizeof(T); }
  bool operator==(const pinned_allocator &) const { return true; }
  bool operator!=(const pinned_allocator &) const { return false; }
};

}  // namespace experimental
}  // namespace cuda
}  // namespace thrust

// .npz reader used to load the expert weight file into pinned host memory.
#pragma once

#include <cstdint>
#include <functional>
#include <string>
#include <vector>

namespace infmoe {

// Called once per member with its name (".npy" stripped) and shape.  Sets *dst to a
// buffer of prod(shape) floats to receive the data, or to nullptr to skip the member.
// A non-zero return aborts the read with that status.
using NpzAllocFn = std::function<int(const std::string& name, const std::vector<int64_t>& shape, float** dst)>;

// threads <= 1: every member's data is read before the next alloc call (a caller may consume it there).
// threads > 1: the walk only hands out destinations; the data is read afterwards by that many threads, each
// with a file descriptor of its own, and is complete when the function returns.
int npz_read(const char* path, const NpzAllocFn& alloc, bool* saw_fortran_order, int threads = 1);

}  // namespace infmoe

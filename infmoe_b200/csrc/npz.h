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

int npz_read(const char* path, const NpzAllocFn& alloc, bool* saw_fortran_order);

}  // namespace infmoe

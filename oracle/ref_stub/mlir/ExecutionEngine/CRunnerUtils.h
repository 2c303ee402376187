// Stand-in for MLIR's mlir/ExecutionEngine/CRunnerUtils.h, which is not in
// this tree (the LLVM/MLIR submodule of the SparseWave reference is not
// vendored).  The reference's benchmark/SparseBenchmarkUtils.cpp uses exactly
// one thing from that header: the ranked memref descriptor, whose five fields
// are fixed by MLIR's C-interface calling convention.  TEST INFRASTRUCTURE.
#pragma once
#include <cstdint>

template <typename T, int N>
struct StridedMemRefType {
  T *basePtr;
  T *data;
  int64_t offset;
  int64_t sizes[N];
  int64_t strides[N];
};

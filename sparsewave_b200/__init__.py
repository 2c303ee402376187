"""sparsewave_b200: B200 (sm_100a) kernels for the SparseWave sparse operators.

The product is `lib/libsparsewave_b200.so` (C ABI in include/sparsewave_b200.h,
built by `python -m sparsewave_b200.build`).  `api` is the thin Python host
layer over it, `sharding` the multi-GPU row-shard layer, `formats` the
benchmark file formats and `workloads` the seeded synthetic inputs.
"""
from .api import (Context, SparseWaveError, chunk_bounds, launch_shape, make_options, partition,
                  row_at_position, shard_rows_by_nnz, validate_options)

__all__ = ["Context", "SparseWaveError", "make_options", "validate_options", "partition", "chunk_bounds",
           "row_at_position", "shard_rows_by_nnz", "launch_shape"]

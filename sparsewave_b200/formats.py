"""On-disk matrix formats of the SparseWave benchmark tooling.

Binary layouts (little endian), as written by benchmark/benchmark_utils.py and
read by benchmark/SparseBenchmarkUtils.cpp in the SparseWave tree:

* ``SWCSR001``: magic, ``<QQQ`` rows/columns/nnz, ``i32[rows+1]`` row offsets,
  ``i32[nnz]`` column indices, ``f32[nnz]`` values
  (benchmark_utils.py:180-211, SparseBenchmarkUtils.cpp:83-124).
* ``SWCOO001``: magic, ``<QQQ``, ``i32[nnz]`` rows, ``i32[nnz]`` columns,
  ``f32[nnz]`` values (benchmark_utils.py:214-237).
* ``SWBSR001``: magic, ``<QQQQQQQ`` padded rows/columns, nnzb, block size,
  original rows/columns/nnz, ``i32[rows/bs+1]`` block-row offsets,
  ``i32[nnzb]`` block columns, ``f32[nnzb*bs*bs]`` block values, then the
  original COO entries ``i32[nnz]``, ``i32[nnz]``, ``f32[nnz]``
  (benchmark_utils.py:315-379, SparseBenchmarkUtils.cpp:142-185).
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np

CSR_MAGIC = b"SWCSR001"
COO_MAGIC = b"SWCOO001"
BSR_MAGIC = b"SWBSR001"
_I32_MAX = (1 << 31) - 1


def write_csr_binary(path, rows: int, cols: int, row_ptr, col_idx, values) -> None:
    row_ptr = np.ascontiguousarray(row_ptr, dtype="<i4")
    col_idx = np.ascontiguousarray(col_idx, dtype="<i4")
    values = np.ascontiguousarray(values, dtype="<f4")
    nnz = len(values)
    if rows > _I32_MAX or nnz > _I32_MAX:
        raise ValueError("matrix rows and NNZ must fit in the i32 CSR type")
    if len(row_ptr) != rows + 1 or len(col_idx) != nnz:
        raise ValueError("CSR arrays have inconsistent sizes")
    with Path(path).open("wb") as f:
        f.write(CSR_MAGIC)
        f.write(struct.pack("<QQQ", rows, cols, nnz))
        f.write(row_ptr.tobytes())
        f.write(col_idx.tobytes())
        f.write(values.tobytes())


def read_csr_binary(path):
    """Returns (rows, cols, row_ptr, col_idx, values)."""
    data = Path(path).read_bytes()
    if data[:8] != CSR_MAGIC:
        raise ValueError("invalid CSR binary header")
    rows, cols, nnz = struct.unpack_from("<QQQ", data, 8)
    off = 32
    need = off + 4 * (rows + 1) + 8 * nnz
    if len(data) < need:
        raise ValueError("could not read CSR arrays: file is truncated")
    row_ptr = np.frombuffer(data, "<i4", rows + 1, off); off += 4 * (rows + 1)
    col_idx = np.frombuffer(data, "<i4", nnz, off); off += 4 * nnz
    values = np.frombuffer(data, "<f4", nnz, off)
    return rows, cols, row_ptr.copy(), col_idx.copy(), values.copy()


def write_coo_binary(path, rows: int, cols: int, row_idx, col_idx, values) -> None:
    row_idx = np.ascontiguousarray(row_idx, dtype="<i4")
    col_idx = np.ascontiguousarray(col_idx, dtype="<i4")
    values = np.ascontiguousarray(values, dtype="<f4")
    if rows > _I32_MAX or cols > _I32_MAX or len(values) > _I32_MAX:
        raise ValueError("matrix dimensions and NNZ must fit in the i32 COO type")
    with Path(path).open("wb") as f:
        f.write(COO_MAGIC)
        f.write(struct.pack("<QQQ", rows, cols, len(values)))
        f.write(row_idx.tobytes())
        f.write(col_idx.tobytes())
        f.write(values.tobytes())


def convert_to_bsr(rows: int, cols: int, row_idx, col_idx, values, block_size: int) -> dict:
    """COO entries -> padded BSR; duplicate coordinates are summed into their
    slot, blocks are ordered by (block row, block column)
    (convert_to_bsr, benchmark_utils.py:240-312)."""
    if block_size <= 0:
        raise ValueError("BSR block size must be positive")
    bs = block_size
    row_idx = np.asarray(row_idx, dtype=np.int64)
    col_idx = np.asarray(col_idx, dtype=np.int64)
    values = np.asarray(values, dtype=np.float64)
    padded_rows = -(-rows // bs) * bs
    padded_cols = -(-cols // bs) * bs
    brows, bcols = padded_rows // bs, padded_cols // bs
    bkey = (row_idx // bs) * max(bcols, 1) + (col_idx // bs)
    uniq, inverse = np.unique(bkey, return_inverse=True)
    nnzb = len(uniq)
    block_values = np.zeros((nnzb, bs, bs), dtype=np.float64)
    np.add.at(block_values, (inverse, row_idx % bs, col_idx % bs), values)
    block_rows = uniq // max(bcols, 1)
    block_cols = uniq % max(bcols, 1)
    brp = np.zeros(brows + 1, dtype=np.int64)
    np.add.at(brp, block_rows + 1, 1)
    brp = np.cumsum(brp)
    occupied = len(np.unique(row_idx * max(padded_cols, 1) + col_idx))
    slots = nnzb * bs * bs
    return {
        "rows": padded_rows, "columns": padded_cols, "original_rows": rows, "original_columns": cols,
        "nnz": len(values), "block_size": bs, "nnzb": nnzb,
        "block_row_offsets": brp.astype(np.int32), "block_column_indices": block_cols.astype(np.int32),
        "block_values": block_values.reshape(-1).astype(np.float32),
        "input_row_indices": row_idx.astype(np.int32), "input_column_indices": col_idx.astype(np.int32),
        "input_values": values.astype(np.float32),
        "block_density": nnzb / (brows * bcols) if brows and bcols else 0.0,
        "internal_zero_fraction": 1.0 - occupied / slots if slots else 0.0,
        "storage_overhead": slots / occupied if occupied else 0.0,
    }


def write_bsr_binary(path, m: dict) -> None:
    for k in ("rows", "columns", "nnzb", "original_rows", "original_columns", "nnz"):
        if m[k] > _I32_MAX:
            raise ValueError("BSR dimensions and NNZ blocks must fit in i32")
    with Path(path).open("wb") as f:
        f.write(BSR_MAGIC)
        f.write(struct.pack("<QQQQQQQ", m["rows"], m["columns"], m["nnzb"], m["block_size"],
                            m["original_rows"], m["original_columns"], m["nnz"]))
        f.write(np.ascontiguousarray(m["block_row_offsets"], "<i4").tobytes())
        f.write(np.ascontiguousarray(m["block_column_indices"], "<i4").tobytes())
        f.write(np.ascontiguousarray(m["block_values"], "<f4").tobytes())
        f.write(np.ascontiguousarray(m["input_row_indices"], "<i4").tobytes())
        f.write(np.ascontiguousarray(m["input_column_indices"], "<i4").tobytes())
        f.write(np.ascontiguousarray(m["input_values"], "<f4").tobytes())


def read_bsr_binary(path) -> dict:
    data = Path(path).read_bytes()
    if data[:8] != BSR_MAGIC:
        raise ValueError("invalid BSR binary header")
    rows, cols, nnzb, bs, orows, ocols, nnz = struct.unpack_from("<QQQQQQQ", data, 8)
    if bs == 0 or rows % bs or cols % bs:
        raise ValueError("BSR dimensions must be divisible by a positive block size")
    if orows > rows or ocols > cols:
        raise ValueError("original BSR dimensions exceed the padded dimensions")
    off = 8 + 7 * 8

    def take(dtype, count):
        nonlocal off
        a = np.frombuffer(data, dtype, count, off).copy()
        off += a.nbytes
        return a

    return {
        "rows": rows, "columns": cols, "nnzb": nnzb, "block_size": bs, "original_rows": orows,
        "original_columns": ocols, "nnz": nnz,
        "block_row_offsets": take("<i4", rows // bs + 1), "block_column_indices": take("<i4", nnzb),
        "block_values": take("<f4", nnzb * bs * bs), "input_row_indices": take("<i4", nnz),
        "input_column_indices": take("<i4", nnz), "input_values": take("<f4", nnz),
    }


def read_matrix_market(path) -> dict:
    """Coordinate Matrix Market file -> entries ordered by (row, column), 0-based; the checks, their order and
    their messages are those of the reference drivers' reader (benchmark_utils.py:56-177): fields real, integer,
    pattern (value 1); symmetry general or symmetric (expanded; square only); blank and comment lines skipped
    anywhere; exactly the expected fields per entry; finite values that fit f32; as many entries as declared.
    Values stay f64 here (`values64`) for the BSR sums; `values` is their f32 rounding."""
    import math
    import struct
    path = Path(path)
    with path.open("r", encoding="utf-8") as f:
        header = f.readline().strip().split()
        if len(header) != 5 or header[:3] != ["%%MatrixMarket", "matrix", "coordinate"]:
            raise ValueError(f"{path}: expected a Matrix Market coordinate matrix")
        field, symmetry = header[3].lower(), header[4].lower()
        if field not in ("real", "integer", "pattern"):
            raise ValueError(f"{path}: unsupported Matrix Market field '{field}'")
        if symmetry not in ("general", "symmetric"):
            raise ValueError(f"{path}: unsupported Matrix Market symmetry '{symmetry}'")
        size_line = next((ln for ln in f if ln.strip() and not ln.lstrip().startswith("%")), None)
        if size_line is None:
            raise ValueError(f"{path}: missing matrix dimensions")
        try:
            rows, cols, declared = map(int, size_line.split())
        except ValueError as error:
            raise ValueError(f"{path}: invalid matrix dimensions") from error
        if rows <= 0 or cols <= 0 or declared < 0:
            raise ValueError(f"{path}: matrix dimensions must be nonnegative")
        if symmetry == "symmetric" and rows != cols:
            raise ValueError(f"{path}: a symmetric matrix must be square")
        entries, read = [], 0
        expected = 2 if field == "pattern" else 3
        for line_number, line in enumerate(f, start=3):
            stripped = line.strip()
            if not stripped or stripped.startswith("%"):
                continue
            parts = stripped.split()
            if len(parts) != expected:
                raise ValueError(f"{path}:{line_number}: expected {expected} fields")
            try:
                r, c = int(parts[0]) - 1, int(parts[1]) - 1
                v = 1.0 if field == "pattern" else (float(int(parts[2])) if field == "integer" else float(parts[2]))
            except ValueError as error:
                raise ValueError(f"{path}:{line_number}: invalid matrix entry") from error
            if not (0 <= r < rows and 0 <= c < cols):
                raise ValueError(f"{path}:{line_number}: matrix index is out of bounds")
            if not math.isfinite(v):
                raise ValueError(f"{path}:{line_number}: matrix value must be finite")
            try:
                struct.pack("<f", v)
            except (OverflowError, struct.error) as error:
                raise ValueError(f"{path}:{line_number}: matrix value must fit in f32") from error
            entries.append((r, c, v))
            read += 1
            if symmetry == "symmetric" and r != c:
                entries.append((c, r, v))
    if read != declared:
        raise ValueError(f"{path}: header declares {declared} entries, but the file contains {read}")
    entries.sort(key=lambda e: (e[0], e[1]))
    values64 = np.array([e[2] for e in entries], np.float64)
    return {"rows": rows, "columns": cols, "row_indices": np.array([e[0] for e in entries], np.int32),
            "column_indices": np.array([e[1] for e in entries], np.int32), "values": values64.astype(np.float32),
            "values64": values64}


def coo_to_csr(rows: int, row_idx, col_idx, values):
    """Stable sort by (row, column); duplicates are kept as separate entries."""
    row_idx = np.asarray(row_idx, np.int64)
    col_idx = np.asarray(col_idx, np.int64)
    order = np.lexsort((col_idx, row_idx))
    rp = np.zeros(rows + 1, np.int64)
    np.add.at(rp, row_idx + 1, 1)
    return (np.cumsum(rp).astype(np.int32), col_idx[order].astype(np.int32),
            np.asarray(values, np.float32)[order])

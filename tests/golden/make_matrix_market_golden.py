"""Generates tests/golden/matrix_market_cases.json from the SparseWave tree's own Matrix Market converter
(benchmark/benchmark_utils.py: read_matrix_market, write_csr_binary, write_coo_binary, convert_to_bsr,
write_bsr_binary), run on the small files below: the exact bytes of the three binary formats, or the error
text.  The tree is found through $SPARSEWAVE_REFERENCE or as a `reference` directory beside this repository.

    python tests/golden/make_matrix_market_golden.py
"""
import json
import os
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
CASES = {
    "unsorted_general_real": "%%MatrixMarket matrix coordinate real general\n% a comment\n4 5 6\n3 2 1.5\n1 5 -2.25\n"
                             "1 1 4\n4 4 0.125\n3 1 7\n2 3 -1e-3\n",
    "symmetric_integer": "%%MatrixMarket matrix coordinate integer symmetric\n3 3 4\n2 1 5\n1 1 2\n3 2 -7\n3 3 1\n",
    "pattern_with_blank_and_comment_lines": "%%MatrixMarket matrix coordinate pattern general\n\n%x\n3 4 3\n3 4\n\n% mid\n1 2\n"
                                            "2 1\n",
    "duplicates_unsorted": "%%MatrixMarket matrix coordinate real general\n4 4 6\n2 2 0.1\n1 1 1e8\n2 2 0.2\n1 1 1.0\n"
                           "1 1 -1e8\n4 3 3\n",
    "odd_shape_bsr_padding": "%%MatrixMarket matrix coordinate real general\n5 3 4\n5 3 1\n1 1 2\n4 2 3\n2 3 4\n",
    "upper_case_header_words": "%%MatrixMarket matrix coordinate REAL General\n2 2 1\n2 1 9\n",
    # malformed inputs
    "extra_field": "%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1 3 4\n",
    "missing_value": "%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1\n",
    "too_few_entries": "%%MatrixMarket matrix coordinate real general\n2 2 3\n1 1 3\n2 2 1\n",
    "too_many_entries": "%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1 3\n2 2 1\n",
    "non_finite_value": "%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1 inf\n",
    "value_beyond_f32": "%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1 1e39\n",
    "symmetric_not_square": "%%MatrixMarket matrix coordinate real symmetric\n2 3 1\n1 1 3\n",
    "zero_rows": "%%MatrixMarket matrix coordinate real general\n0 3 0\n",
    "skew_symmetric": "%%MatrixMarket matrix coordinate real skew-symmetric\n2 2 1\n2 1 3\n",
    "array_layout": "%%MatrixMarket matrix array real general\n2 2\n1\n2\n3\n4\n",
    "complex_field": "%%MatrixMarket matrix coordinate complex general\n2 2 1\n1 1 3 4\n",
    "index_out_of_bounds": "%%MatrixMarket matrix coordinate real general\n2 2 1\n3 1 3\n",
    "bad_dimensions": "%%MatrixMarket matrix coordinate real general\n2 x 1\n1 1 3\n",
    "no_dimensions": "%%MatrixMarket matrix coordinate real general\n% only a comment\n",
    "bad_entry": "%%MatrixMarket matrix coordinate real general\n2 2 1\n1 one 3\n",
}
BLOCK_SIZE = 2


def main():
    root = os.environ.get("SPARSEWAVE_REFERENCE") or str(HERE.parents[2] / "reference")
    sys.path.insert(0, str(Path(root) / "benchmark"))
    import benchmark_utils as ref
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        for name, text in CASES.items():
            mtx = tmp / "m.mtx"
            mtx.write_text(text)
            try:
                m = ref.read_matrix_market(mtx)
                ref.write_csr_binary(tmp / "o.csr", m)
                ref.write_coo_binary(tmp / "o.coo", m)
                ref.write_bsr_binary(tmp / "o.bsr", ref.convert_to_bsr(m, BLOCK_SIZE))
                out[name] = {"text": text, "csr": (tmp / "o.csr").read_bytes().hex(),
                             "coo": (tmp / "o.coo").read_bytes().hex(), "bsr": (tmp / "o.bsr").read_bytes().hex()}
            except ValueError as error:
                out[name] = {"text": text, "error": str(error).replace(str(mtx), "<path>")}
    (HERE / "matrix_market_cases.json").write_text(json.dumps({"block_size": BLOCK_SIZE, "cases": out}, indent=1))
    for name, c in out.items():
        print(name, "->", c.get("error", f"{len(c.get('csr', '')) // 2} csr bytes"))


if __name__ == "__main__":
    main()

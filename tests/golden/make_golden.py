"""Writes ``reference_fixtures.json``: the known-answer cases of the reference's own gtest
files, transcribed from their source text (the reference cannot run without a GPU, and its
tests are the only fixtures it owns for this path).

  colwise_slicing   tests/test_colwise_slicing.cc:7-21
  colwise_sampling  tests/test_colwise_sampling.cc:7-60
  rowwise_slicing   tests/test_rowwise_slicing.cc:7-25
  walks             tests/test_random_walk.cc:28-61, tests/test_node2vec.cc:28-61

Run: python tests/golden/make_golden.py
"""
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    indptr = [5 * i for i in range(21)]
    indices = list(range(100))
    fx = {
        "colwise_slicing": {
            "indptr": indptr, "indices": indices, "cols": [0, 1, 2],
            "expect_indptr": [0, 5, 10, 15], "expect_indices": list(range(15)),
        },
        "colwise_sampling": {
            "indptr": indptr, "indices": indices,
            "copy_all": {"fanout": 6, "replace": False,
                         "expect_indptr": indptr, "expect_indices": indices},
            "replace": [{"fanout": 6, "expect_indptr": [6 * i for i in range(21)]},
                        {"fanout": 4, "expect_indptr": [4 * i for i in range(21)]}],
        },
        "rowwise_slicing": {
            # indptr = cat(zeros(10), arange(3)*2); indices = arange(5,7).repeat(2)
            "indptr": [0] * 10 + [0, 2, 4], "indices": [5, 6, 5, 6], "rows": [5],
            # sliced on CSR: one row kept, its entries are columns 10 and 11
            "expect_csr_indptr_numel": 2, "expect_csr_indices": [10, 11],
        },
        "walks": {
            # the reference test builds a 5-entry indptr blob out of 6 written values; the
            # graph below is the well-formed 5-node graph those values describe
            "indptr": [0, 0, 1, 2, 3, 5], "indices": [0, 1, 1, 2, 3],
            "seeds": [4, 2, 3, 1], "walk_length": 3, "p": 2.0, "q": 0.5,
            "invariant": "every consecutive pair (a,b) of a trace has b in column a, or b == -1",
        },
    }
    with open(os.path.join(HERE, "reference_fixtures.json"), "w") as f:
        json.dump(fx, f, indent=1)


if __name__ == "__main__":
    main()

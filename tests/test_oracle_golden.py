"""Pins the CPU oracle to the reference: every golden vector under tests/golden/ was produced by
the reference implementation's own code, and the oracle must reproduce each one byte for byte."""

import hashlib
import json
import os

import pytest

import cases
import mlf_oracle as oracle


def _load(golden_dir, name):
    with open(os.path.join(golden_dir, name)) as f:
        return json.load(f)


def test_header_bytes_match_reference(golden_dir):
    rows = _load(golden_dir, "headers.json")
    assert len(rows) == len(cases.HEADER_MATRIX)
    for row in rows:
        name = row["dtype"].split(".")[-1]
        assert oracle.header_bytes(name, row["shape"]).hex() == row["hex"], row


def test_header_parse_round_trip(golden_dir):
    for row in _load(golden_dir, "headers.json"):
        raw = bytes.fromhex(row["hex"])
        name, shape, used = oracle.parse_header(raw + b"tail")
        assert name == row["dtype"].split(".")[-1]
        assert list(shape) == row["shape"]
        assert used == len(raw)


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_objects_match_reference(golden_dir, name):
    gold = _load(golden_dir, f"{name}.json")
    produced = oracle.save_case(cases.CASES[name]())
    assert [p[0] for p in produced] == [o["name"] for o in gold["objects"]]
    records = []
    for (obj_name, data, recs), g in zip(produced, gold["objects"]):
        assert len(data) == g["size"]
        if "file" in g:
            with open(os.path.join(golden_dir, g["file"]), "rb") as f:
                assert data == f.read()
        else:
            assert data[: 4096 + 512].hex() == g["head_hex"]
        assert hashlib.sha256(data).hexdigest() == g["sha256"]
        # bucket order: tensors first, then blobs
        assert [r[0] for r in recs] == [i["fqn"] for i in g["item_order"]]
        records += [(obj_name, off, length, fqn) for fqn, off, length in recs]
    records.sort()
    want = [(w["relative_path"], w["offset"], w["length"], w["index"]["fqn"]) for w in gold["write_results"]]
    assert records == want
    assert all(w["size_in_bytes"] == w["length"] for w in gold["write_results"])


def test_narrow_reads_match_reference(golden_dir):
    rows = _load(golden_dir, "narrow.json")
    tensors = {f"n.{i}": cases.narrow_source(i) for i in range(len(cases.NARROW_CASES))}
    ((_, data, recs),) = oracle.save_case({"tensors": tensors, "blobs": {}, "bucket_count": 1})
    where = {fqn: (off, length) for fqn, off, length in recs}
    for row in rows:
        off, length = where[f"n.{row['i']}"]
        dtype_name, got = oracle.read_item(data, off, length, row["storage_offsets"], row["lengths"])
        assert dtype_name == row["dtype"].split(".")[-1]
        assert got.hex() == row["hex"], row["i"]


def test_bucket_split_known_answers():
    # one bin keeps plan order
    items = [("a", False, 10), ("b", True, 0), ("c", False, 30)]
    assert oracle.split_by_size_and_type(1, items) == [[0, 1, 2]]
    # blobs round-robin first; tensors largest first to the lightest bucket, ties to the lowest index
    items = [("t0", False, 5), ("b0", True, 0), ("t1", False, 9), ("b1", True, 0), ("t2", False, 5), ("b2", True, 0)]
    assert oracle.split_by_size_and_type(2, items) == [[1, 5, 2], [3, 0, 4]]

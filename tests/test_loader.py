"""Loading partitions from disk: the parallel text reader against numpy's, the reference's three text formats, and
the binary partition format (whole partition and one rank's view)."""
import os
import time

import numpy as np
import pytest

import drone_b200 as db
from drone_b200 import graphgen as gg
from drone_b200 import partition as pt


def test_text_reader_handles_ragged_input(tmp_path):
    path = tmp_path / "ragged.txt"
    path.write_bytes(b"3 4\r\n\n   \n5\t-6   7\n+8 9")            # CRLF, blank lines, tabs, signs, no final newline
    values, lines = pt.read_text_ints(str(path), with_lines=True)
    assert values.tolist() == [3, 4, 5, -6, 7, 8, 9]
    assert lines.tolist() == [0, 2, 5, 7]
    assert pt.read_text_ints(str(path)).tolist() == values.tolist()
    empty = tmp_path / "empty.txt"
    empty.write_bytes(b"")
    values, lines = pt.read_text_ints(str(empty), with_lines=True)
    assert len(values) == 0 and lines.tolist() == [0]
    odd = tmp_path / "odd.txt"
    odd.write_text("1 2\n3\n")
    with pytest.raises(ValueError, match="odd number"):
        pt.read_edge_list(str(odd))
    for bad in (b"1 2\n3 x\n", b"1 99999999999\n", b"4 -\n"):
        (tmp_path / "bad.txt").write_bytes(bad)
        with pytest.raises(db.DroneError, match="byte"):
            pt.read_text_ints(str(tmp_path / "bad.txt"))
    with pytest.raises(db.DroneError, match="cannot open"):
        pt.read_text_ints(str(tmp_path / "missing.txt"))


def test_text_reader_matches_numpy_on_a_file_cut_into_pieces(tmp_path):
    """Above 1 MB the file is parsed in pieces by several threads; values and line starts must come out in file order."""
    rng = np.random.default_rng(3)
    rows = rng.integers(0, 2**31 - 1, size=(300_000, 2), dtype=np.int64)
    path = str(tmp_path / "edges.txt")
    np.savetxt(path, rows, fmt="%d")
    assert os.path.getsize(path) > (1 << 20)
    t0 = time.perf_counter()
    u, v = pt.read_edge_list(path)
    fast = time.perf_counter() - t0
    assert np.array_equal(u, rows[:, 0]) and np.array_equal(v, rows[:, 1])
    values, lines = pt.read_text_ints(path, with_lines=True)
    assert np.array_equal(lines, np.arange(0, 2 * len(rows) + 1, 2))
    t0 = time.perf_counter()
    slow = np.loadtxt(path, dtype=np.int64)
    numpy_time = time.perf_counter() - t0
    assert np.array_equal(slow, rows)
    assert fast < numpy_time                      # the point of the exercise (typically 20-50x)


@pytest.mark.parametrize("parts", [1, 3, 8])
def test_partition_files_and_binary_round_trip(tmp_path, parts):
    n, u, v = gg.rmat_graph(10, 8, seed=13, self_loops="add")
    part = pt.ebv_partition(n, u.numpy(), v.numpy(), parts)
    part.write_files(str(tmp_path / "text"))
    back = pt.read_partition_files(str(tmp_path / "text"), n, parts)
    for p in range(parts):
        assert np.array_equal(back.part_u[p], part.part_u[p]) and np.array_equal(back.part_v[p], part.part_v[p])
    assert np.array_equal(back.replicas, part.replicas)
    shared = part.replicas > 1
    assert np.array_equal(back.owner[shared], part.owner[shared])

    path = str(tmp_path / "part.bin")
    pt.save_partition(part, path)
    whole = pt.load_partition(path)
    assert whole.n_vertices == n and whole.n_parts == parts
    for p in range(parts):
        assert np.array_equal(whole.part_u[p], part.part_u[p]) and np.array_equal(whole.part_v[p], part.part_v[p])
    assert np.array_equal(whole.owner, part.owner) and np.array_equal(whole.replicas, part.replicas)
    assert np.array_equal(whole.presence_bits(), part.presence_bits())
    for p in range(parts):                        # one rank's view builds the same local graph and routing tables
        mine = pt.load_partition(path, part=p)
        assert all(mine.part_u[q] is None for q in range(parts) if q != p)
        a, b = mine.local_graph(p), part.local_graph(p)
        for name in ("l2g", "index", "dst", "master_worker_index", "master2workers", "mirror2worker"):
            assert np.array_equal(getattr(a, name), getattr(b, name)), name


def test_binary_format_rejects_damaged_files(tmp_path):
    n, u, v = gg.rmat_graph(8, 4, seed=2, self_loops="add")
    part = pt.ebv_partition(n, u.numpy(), v.numpy(), 2)
    path = str(tmp_path / "p.bin")
    pt.save_partition(part, path)
    data = open(path, "rb").read()
    open(path, "wb").write(b"NOTAPART" + data[8:])
    with pytest.raises(db.DroneError, match="magic"):
        pt.load_partition(path)
    open(path, "wb").write(data[:len(data) - 100])
    with pytest.raises(db.DroneError, match="shorter"):
        pt.load_partition(path)
    open(path, "wb").write(data)
    with pytest.raises(db.DroneError, match="part 5"):
        pt.load_partition(path, part=5)

"""What a step looks like to the parts, checked on the CPU: the attention mixer's cut of the rows into query runs,
and the one copy that carries the step's int32 arrays (every array on a 16-byte boundary)."""
import numpy as np
import torch

from garlic_inference_b200.engine.step import _Staging
from garlic_inference_b200.parts import StepShape
from garlic_inference_b200.parts.attention import query_runs


def _shape(lens, past, slots=None):
    starts, row = [], 0
    for n in lens:
        starts.append(row)
        row += n
    return StepShape(slots or list(range(len(lens))), starts, list(lens), list(past), all(n == 1 for n in lens))


def test_query_runs_cover_every_row_once_and_never_cross_a_sequence():
    lens, past = [1, 37, 150, 64, 3, 129, 128, 200], [0, 10, 0, 64, 500, 1, 128, 77]
    shape = _shape(lens, past, slots=[5, 2, 9, 0, 1, 7, 3, 4])
    for rows in (64, 128, 16):
        runs = query_runs(shape, rows)
        assert runs.dtype == np.int32 and runs.shape[1] == 4
        covered = np.zeros(sum(lens), dtype=int)
        for slot, row0, n, pos0 in runs.tolist():
            i = shape.seq_slots.index(slot)
            assert 1 <= n <= rows
            assert shape.seq_starts[i] <= row0 and row0 + n <= shape.seq_starts[i] + lens[i], "a run crosses a sequence"
            assert pos0 == past[i] + (row0 - shape.seq_starts[i]), "the run's first position follows from its first row"
            covered[row0:row0 + n] += 1
        assert (covered == 1).all(), "every row in exactly one run"
        assert len(runs) == sum(-(-n // rows) for n in lens)
        keys = [p + n for _, _, n, p in runs.tolist()]
        assert keys == sorted(keys, reverse=True), "the runs with the most keys to walk come first"
    assert query_runs(_shape([], []), 64).shape == (0, 4)


def test_one_copy_carries_the_steps_arrays_each_on_a_16_byte_boundary():
    st = _Staging(torch.device("cpu"))
    arrays = [np.arange(5, dtype=np.int32), np.arange(12, dtype=np.int32).reshape(3, 4).reshape(-1),
              np.zeros(0, dtype=np.int32), np.arange(7, dtype=np.int32) * 3]
    out = st.upload(arrays)
    base = st.dev.data_ptr()
    for a, t in zip(arrays, out):
        assert t.dtype == torch.int32 and t.numel() == a.size and t.tolist() == a.tolist()
        assert (t.data_ptr() - base) % 16 == 0
    assert st.bytes_uploaded == 4 * (8 + 12 + 0 + 8)          # sizes rounded up to whole 16-byte pieces
    again = st.upload([np.arange(3, dtype=np.int32)])           # the buffers are used again
    assert again[0].tolist() == [0, 1, 2] and again[0].data_ptr() == base
    big = st.upload([np.arange(5000, dtype=np.int32)])          # and grow when a step needs more
    assert big[0].numel() == 5000 and st.capacity >= 5000 and int(big[0][-1]) == 4999

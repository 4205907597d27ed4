"""``SequenceBatch`` / ``Seq2SeqBatch`` shifting for padded and packed batches and the accumulating data reader
(cf. fairseq2 ``datasets/batch.py:160-212``, ``datasets/data_reader.py:74-170``)."""
from __future__ import annotations

import pytest
import torch

from fairseq2_b200.data import read_sequence
from fairseq2_b200.datasets.batch import Seq2SeqBatch, SequenceBatch
from fairseq2_b200.datasets.data_reader import DataPipelineReader
from fairseq2_b200.gang import FakeGang


def test_padded_auto_regressive_shift() -> None:
    seqs = torch.tensor([[1, 2, 3, 4], [5, 6, 0, 0]])
    mask = torch.tensor([[False, True, True, True], [False, False, False, False]])
    batch = SequenceBatch(seqs, [4, 2], target_mask=mask)
    assert batch.padding == 2 and batch.num_elements == 6 and batch.num_target_elements == 3
    inp, tgt = batch.as_auto_regressive()
    assert inp.seqs.tolist() == [[1, 2, 3], [5, 6, 0]] and tgt.seqs.tolist() == [[2, 3, 4], [6, 0, 0]]
    assert inp.seq_lens == [3, 1] and tgt.seq_lens == [3, 1]
    assert tgt.target_mask.tolist() == [[True, True, True], [False, False, False]]
    x, layout = inp.as_input()
    assert x is inp.seqs and list(layout.seq_lens) == [3, 1] and layout.padded and not layout.packed
    with pytest.raises(ValueError):
        SequenceBatch(torch.zeros(2, 1, dtype=torch.long), [1, 1]).as_auto_regressive()
    with pytest.raises(ValueError):
        SequenceBatch(seqs, [4])


def test_packed_auto_regressive_trims_the_last_sequence() -> None:
    seqs = torch.arange(1, 8)                                 # documents [1 2 3] [4 5 6 7]
    batch = SequenceBatch(seqs, [3, 4], packed=True)
    inp, tgt = batch.as_auto_regressive()
    assert inp.seqs.tolist() == [1, 2, 3, 4, 5, 6] and tgt.seqs.tolist() == [2, 3, 4, 5, 6, 7]
    assert inp.seq_lens == [3, 3] and inp.packed
    one = SequenceBatch(torch.arange(4), [3, 1], packed=True).as_auto_regressive()[0]
    assert one.seq_lens == [3]                                # a trailing one-token document disappears
    padded = SequenceBatch(torch.arange(6), [3, 2], packed=True)   # one padding slot at the end
    assert padded.padding == 1 and padded.as_auto_regressive()[0].seq_lens == [3, 2]
    _, layout = inp.as_input()
    assert layout.packed and list(layout.seq_begin_indices)[:2] == [0, 3]


def test_seq2seq_batch_shifts_the_target_only() -> None:
    b = Seq2SeqBatch(torch.ones(2, 5, 3), [5, 4], torch.tensor([[9, 1, 2, 3], [9, 4, 5, 0]]), [4, 3])
    inp, tgt = b.as_auto_regressive()
    assert inp.source.seqs.shape == (2, 5, 3) and inp.target.seqs.tolist() == [[9, 1, 2], [9, 4, 5]]
    assert tgt.seqs.tolist() == [[1, 2, 3], [4, 5, 0]] and tgt.seq_lens == [3, 2]


def test_reader_accumulates_and_drops_the_remainder() -> None:
    gang = FakeGang(torch.device("cpu"))
    pipeline = read_sequence(list(range(7))).and_return()
    reader = DataPipelineReader("d", "train", pipeline, gang, num_accumulate=3, drop_remainder=True)
    assert list(reader) == [[0, 1, 2], [3, 4, 5]]
    reader.reset()
    keep = DataPipelineReader("d", "train", read_sequence(list(range(7))).and_return(), gang, num_accumulate=3,
                              drop_remainder=False)
    assert list(keep) == [[0, 1, 2], [3, 4, 5], [6]]
    state_reader = DataPipelineReader("d", "train", read_sequence(list(range(9))).and_return(), gang, num_accumulate=2)
    it = iter(state_reader)
    assert next(it) == [0, 1]
    state = state_reader.state_dict()
    assert next(it) == [2, 3]
    state_reader.load_state_dict(state)
    assert next(iter(state_reader)) == [2, 3]

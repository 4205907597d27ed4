"""Lazy, Lookup, pad_seqs and the pickle wrapper for plain iterators."""
from __future__ import annotations

import pickle

import pytest
import torch

from fairseq2_b200.data.utils import IteratorPickleWrapper, read_pickle_wrapped_iterator
from fairseq2_b200.nn.utils.padding import pad_seqs
from fairseq2_b200.runtime.dependency import DependencyContainer
from fairseq2_b200.runtime.lazy import Lazy
from fairseq2_b200.runtime.lookup import MappingLookup, ResolverLookup


def test_lazy_builds_once() -> None:
    calls: list[int] = []
    lazy = Lazy(lambda: calls.append(1) or [1, 2, 3])
    assert calls == []
    assert lazy.get() is lazy.get() and calls == [1]


def test_lookups() -> None:
    m = MappingLookup(int, {"a": 1})
    assert m.maybe_get("a") == 1 and m.maybe_get("b") is None and list(m.iter_keys()) == ["a"] and m.kls is int
    with pytest.raises(LookupError):
        m.get("b")
    c = DependencyContainer()
    c.register_instance(str, "x", key="k1")
    c.register_instance(str, "y", key="k2")
    r = ResolverLookup(c, str)
    assert sorted(r.iter_keys()) == ["k1", "k2"] and r.get("k2") == "y" and r.maybe_get("zz") is None


def test_pad_seqs() -> None:
    seqs = [torch.arange(3), torch.arange(5), torch.arange(1)]
    out, layout = pad_seqs(seqs, pad_value=-1, pad_to_multiple=4)
    assert out.shape == (3, 8)
    assert out[0].tolist() == [0, 1, 2, -1, -1, -1, -1, -1]
    assert list(layout.seq_lens) == [3, 5, 1] and layout.padded
    feats, _ = pad_seqs([torch.ones(2, 4), torch.ones(3, 4)])
    assert feats.shape == (2, 3, 4) and float(feats[0, 2].sum()) == 0.0
    with pytest.raises(ValueError):
        pad_seqs([torch.ones(2, 4), torch.ones(3, 5)])
    with pytest.raises(ValueError):
        pad_seqs([])


def _numbers():  # type: ignore[no-untyped-def]
    yield from range(6)


def test_iterator_pickle_wrapper_keeps_position() -> None:
    it = IteratorPickleWrapper(_numbers)
    assert [next(it), next(it)] == [0, 1]
    clone = pickle.loads(pickle.dumps(it))
    assert list(clone) == [2, 3, 4, 5]


def test_read_pickle_wrapped_iterator_state_dict() -> None:
    pipeline = read_pickle_wrapped_iterator(_numbers).and_return()
    it = iter(pipeline)
    assert [next(it), next(it), next(it)] == [0, 1, 2]
    state = pipeline.state_dict()
    assert list(it) == [3, 4, 5]
    pipeline.load_state_dict(state)
    assert list(pipeline) == [3, 4, 5]
    pipeline.reset()
    assert list(pipeline) == [0, 1, 2, 3, 4, 5]


def test_recipe_dataset_and_tokenizer_wrappers() -> None:
    from fairseq2_b200.data.tokenizers.char import CharTokenizer
    from fairseq2_b200.recipe import RecipeDataset, RecipeTokenizer

    ds = RecipeDataset([1, 2], {"a": 1}, "family")
    assert ds.as_(list) == [1, 2] and ds.config == {"a": 1} and ds.family == "family"
    with pytest.raises(TypeError, match="expected to be of type"):
        ds.as_(dict)
    inner = CharTokenizer()
    tok = RecipeTokenizer(inner, None, "char")
    assert tok.as_(CharTokenizer) is inner and tok.vocab_info == inner.vocab_info
    ids = tok.create_encoder()("ab")
    assert tok.create_decoder()(ids[1:-1]) == "ab" and tok.create_raw_encoder()("ab").tolist() == ids[1:-1].tolist()
    with pytest.raises(TypeError):
        tok.as_(dict)

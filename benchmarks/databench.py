"""Host-side throughput of the native data pipeline: text -> SentencePiece ids -> length buckets -> collated batches.

    python -m benchmarks.databench [--lines 200000] [--workers 1 2 4 8]

Trains a small SentencePiece model on synthetic text (with the ``sentencepiece`` package, which is only needed for
that), then times three ways of tokenizing inside ``DataPipeline.map``: the package's encoder called through Python
(every call takes the interpreter lock), and the toolkit's native encoder with 1..N worker threads (no lock). Prints
one JSON line per case with lines/s and tokens/s. The last cases use ``map(..., deterministic=False)``: results in the
order in which the workers finish them.
"""
from __future__ import annotations

import argparse
import io
import json
import random
import tempfile
import time
from pathlib import Path

import torch


def _corpus(n: int, seed: int = 0) -> list[str]:
    rng = random.Random(seed)
    syll = ["ka", "to", "mi", "ren", "sol", "ve", "dra", "qui", "an", "or", "est", "ing", "pre", "con", "tion", "ly"]
    words = ["".join(rng.choice(syll) for _ in range(rng.randint(1, 4))) for _ in range(5000)]
    return [" ".join(rng.choice(words) for _ in range(rng.randint(5, 60))) for _ in range(n)]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--lines", type=int, default=200_000)
    ap.add_argument("--workers", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--vocab", type=int, default=8000)
    args = ap.parse_args()

    import sentencepiece as spm

    from fairseq2_b200.data.data_pipeline import Collater
    from fairseq2_b200.data.text.reader import read_text
    from fairseq2_b200.data.tokenizers.sentencepiece import SentencePieceEncoder, SentencePieceModel

    lines = _corpus(args.lines)
    with tempfile.TemporaryDirectory() as tmp:
        text_path = Path(tmp) / "corpus.txt"
        text_path.write_text("\n".join(lines) + "\n")
        blob = io.BytesIO()
        spm.SentencePieceTrainer.train(sentence_iterator=iter(lines[:50_000]), model_writer=blob, vocab_size=args.vocab,
                                       model_type="unigram", hard_vocab_limit=False, minloglevel=2)
        model_path = Path(tmp) / "m.model"
        model_path.write_bytes(blob.getvalue())
        package = spm.SentencePieceProcessor(model_file=str(model_path))
        native = SentencePieceEncoder(SentencePieceModel(model_path)).native

        def package_encode(line: str) -> torch.Tensor:
            return torch.tensor(package.EncodeAsIds(line), dtype=torch.int64)

        def run(name: str, fn, workers: int, ordered: bool = True) -> None:  # type: ignore[no-untyped-def]
            pipeline = (read_text(text_path, rtrim=True).map(fn, num_parallel_calls=workers, deterministic=ordered)
                        .bucket(64).map(Collater(pad_value=0)).prefetch(4).and_return())
            t0 = time.perf_counter()
            tokens = batches = 0
            for batch in pipeline:
                tokens += sum(batch["seq_lens"]) if isinstance(batch, dict) else 0
                batches += 1
            dt = time.perf_counter() - t0
            print(json.dumps({"case": name, "workers": workers, "lines": len(lines), "batches": batches,
                              "seconds": round(dt, 3), "lines_per_s": round(len(lines) / dt),
                              "tokens_per_s": round(tokens / dt)}), flush=True)

        run("package encoder through Python", package_encode, 1)
        run("package encoder through Python", package_encode, max(args.workers))
        for w in args.workers:
            run("native encoder", native, w)
        for w in args.workers:
            if w > 1:
                run("native encoder, results in completion order", native, w, ordered=False)


if __name__ == "__main__":
    main()

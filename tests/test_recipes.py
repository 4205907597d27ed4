"""End-to-end recipe runs on CPU with the tiny LLaMA and the byte-level tokenizer."""
import json
import math
from pathlib import Path

import pytest
import torch

from fairseq2_b200.recipe.cli import main


def _write_sft_data(root: Path, n: int = 64) -> Path:
    d = root / "data"
    (d / "train").mkdir(parents=True)
    (d / "valid").mkdir(parents=True)
    for split in ("train", "valid"):
        with open(d / split / "part0.jsonl", "w") as fp:
            for i in range(n if split == "train" else 8):
                fp.write(json.dumps({"id": i, "src": f"Q: what is {i} plus {i}? ", "tgt": f"A: {2 * i}."}) + "\n")
    return d


def _sft_args(tmp_path: Path, data: Path, extra: list[str]) -> list[str]:
    src = f"[{{path: {data}, split: train}}]"
    vsrc = f"[{{path: {data}, split: valid}}]"
    return [str(tmp_path / "out"), "--no-sweep-dir", "--no-exit-on-error", "--config",
            "model.name=null", "model.family=llama", "model.arch=tiny", "tokenizer.name=char_tokenizer",
            f"dataset.config_overrides={{sources: {{train: {src}, valid: {vsrc}}}}}",
            "dataset.max_seq_len=128", "dataset.max_num_tokens=256", "dataset.valid_split=valid",
            "trainer.mixed_precision.mode=off", "optimizer.config.lr=1e-3",
            "lr_scheduler.config.num_warmup_steps=1", "regime.validate_every_n_steps=2",
            "regime.checkpoint_every_n_steps=2", "regime.publish_metrics_every_n_steps=1",
            "regime.export_hugging_face=false", "common.metric_recorders.jsonl=true", *extra]


@pytest.mark.parametrize("packed", [True, False])
def test_lm_sft_recipe_end_to_end(tmp_path: Path, packed: bool) -> None:
    from recipes.lm.sft.recipe import LMSFTRecipe

    data = _write_sft_data(tmp_path)
    args = _sft_args(tmp_path, data, ["regime.num_steps=4", f"dataset.packed={str(packed).lower()}"])
    assert main(LMSFTRecipe(), args) == 0
    out = tmp_path / "out"
    assert (out / "config.yaml").exists()
    assert (out / "logs" / "rank_0.log").exists()
    assert (out / "checkpoints" / "step_4").is_dir()
    lines = [json.loads(l) for l in open(out / "metrics" / "train.jsonl")]
    assert len(lines) == 4 and all("NLL Loss" in l for l in lines)
    assert lines[-1]["NLL Loss"] < lines[0]["NLL Loss"]
    assert (out / "metrics" / "valid.jsonl").exists()
    # resume: two more steps continue from step 4
    args = _sft_args(tmp_path, data, ["regime.num_steps=6", f"dataset.packed={str(packed).lower()}"])
    assert main(LMSFTRecipe(), args) == 0
    lines = [json.loads(l) for l in open(out / "metrics" / "train.jsonl")]
    assert [l["Step"] for l in lines][-2:] == [5, 6]


def test_dump_config(capsys: pytest.CaptureFixture[str]) -> None:
    from recipes.lm.sft.recipe import LMSFTRecipe

    assert main(LMSFTRecipe(), ["--dump-config", "--config", "regime.num_steps=7"]) == 0
    out = capsys.readouterr().out
    assert "num_steps: 7" in out and "data_parallelism: fsdp" in out


def test_bad_config_exit_code() -> None:
    from recipes.lm.sft.recipe import LMSFTRecipe

    assert main(LMSFTRecipe(), ["--dump-config", "--config", "regime.num_stepz=7"]) != 0


def test_lm_train_recipe(tmp_path: Path) -> None:
    from recipes.lm.train.recipe import LMTrainRecipe

    d = tmp_path / "corpus"
    d.mkdir()
    with open(d / "shard0.jsonl", "w") as fp:
        for i in range(200):
            fp.write(json.dumps({"text": f"document {i}: " + "the quick brown fox jumps over the lazy dog. " * (1 + i % 5)}) + "\n")
    args = [str(tmp_path / "out"), "--no-sweep-dir", "--no-exit-on-error", "--config", "model.arch=tiny",
            "tokenizer.name=char_tokenizer", f"dataset.config_overrides={{sources: [{{path: {d}}}]}}",
            "dataset.max_seq_len=128", "dataset.max_num_tokens=512", "trainer.mixed_precision.mode=off",
            "optimizer.config.lr=1e-3", "lr_scheduler.config.num_warmup_steps=1", "regime.num_steps=4",
            "regime.checkpoint_every_n_steps=4", "regime.publish_metrics_every_n_steps=1",
            "common.metric_recorders.jsonl=true"]
    assert main(LMTrainRecipe(), args) == 0
    lines = [json.loads(l) for l in open(tmp_path / "out" / "metrics" / "train.jsonl")]
    assert len(lines) == 4 and lines[-1]["NLL Loss"] < lines[0]["NLL Loss"]
    assert all(l["Number of Elements"] == 512 for l in lines)       # packed buffers are always full


def test_lm_generate_recipe(tmp_path: Path) -> None:
    from recipes.lm.generate.recipe import LMGenerateRecipe

    prompts = tmp_path / "prompts.jsonl"
    with open(prompts, "w") as fp:
        for i in range(5):
            fp.write(json.dumps({"id": f"p{i}", "prompt": f"Question {i}?"}) + "\n")
    for gen in ("sampling", "beam_search"):
        out = tmp_path / gen
        args = [str(out), "--no-sweep-dir", "--no-exit-on-error", "--config", "model.name=null", "model.family=llama",
                "model.arch=tiny", "model.dtype=float32", "tokenizer.name=char_tokenizer",
                f"dataset.config_overrides={{path: {prompts}}}", "dataset.batch_size=2",
                f"seq_generator.name={gen}", "seq_generator.config={max_gen_len: 8}"]
        assert main(LMGenerateRecipe(), args) == 0
        rows = [json.loads(l) for l in open(out / "output" / "rank_0.jsonl")]
        assert [r["id"] for r in rows] == [f"p{i}" for i in range(5)]
        assert all(1 <= len(r["token_indices"]) <= 8 + 20 for r in rows)
        assert "<<<<< RESPONSE >>>>>" in (out / "output" / "rank_0.txt").read_text()


def test_sft_recipe_exports_hugging_face_checkpoint(tmp_path: Path) -> None:
    """The out-of-process exporter writes ``step_N/hg`` which loads into ``transformers`` with equal logits."""
    transformers = pytest.importorskip("transformers")
    from recipes.lm.sft.recipe import LMSFTRecipe

    data = _write_sft_data(tmp_path, 16)
    args = [a for a in _sft_args(tmp_path, data, ["regime.num_steps=2", "dataset.packed=true"])
            if a != "regime.export_hugging_face=false"] + ["regime.export_hugging_face=true",
                                                           "regime.save_model_only=false"]
    assert main(LMSFTRecipe(), args) == 0
    hg = tmp_path / "out" / "checkpoints" / "step_2" / "hg"
    assert (hg / "config.json").exists() and (hg / "model.safetensors").exists(), \
        (tmp_path / "out" / "checkpoints" / "step_2" / "hg.stderr").read_text()
    hf = transformers.AutoModelForCausalLM.from_pretrained(hg, torch_dtype=torch.float32).eval()

    from fairseq2_b200.gang import create_fake_gangs
    from fairseq2_b200.models.family import get_model_family
    from fairseq2_b200.nn.batch_layout import BatchLayout

    fam = get_model_family("llama")
    cfg = fam.get_arch_config("tiny")
    g = create_fake_gangs(torch.device("cpu"))
    ours = fam.create_new_model(cfg, g)
    fam.load_into(ours, tmp_path / "out" / "checkpoints" / "step_2" / "model", cfg, g)
    x = torch.randint(1, 300, (1, 12))
    with torch.no_grad():
        a = ours.eval()(x, BatchLayout((1, 12), [12]))
        b = hf(x).logits
    assert torch.allclose(a, b, atol=5e-2), float((a - b).abs().max())


def test_chatbot_program_streams_reply() -> None:
    from fairseq2_b200.data.tokenizers import CharTokenizer
    from fairseq2_b200.gang import FakeGang, create_fake_gangs
    from fairseq2_b200.generation import SamplingSequenceGenerator, TopKSampler
    from fairseq2_b200.models.family import get_model_family
    from recipes.chatbot.chatbot import LLaMADialogEncoder, Message, MistralDialogEncoder, StandardChatbot
    from recipes.chatbot.program import ChatbotProgram, ProgramView

    torch.manual_seed(0)
    dev = torch.device("cpu")
    tok = CharTokenizer()
    fam = get_model_family("llama")
    model = fam.create_new_model(fam.get_arch_config("tiny"), create_fake_gangs(dev)).eval()
    vi = tok.vocab_info
    gen = SamplingSequenceGenerator(model, vi.eos_idx, vi.pad_idx, TopKSampler(1), max_gen_len=6)
    enc = LLaMADialogEncoder(tok, dev)
    ids = enc.encode([Message("system", "be brief"), Message("user", "hi"), Message("bot", "hello"), Message("user", "bye?")])
    assert ids[0] == vi.bos_idx and (ids == vi.eos_idx).sum() == 1
    assert not MistralDialogEncoder(tok, dev).supports_system_prompt

    class View(ProgramView):
        def __init__(self) -> None:
            self.inputs, self.pieces = iter(["hi there", "bye"]), []

        def input_system_prompt(self) -> str:
            return ""

        def input_message(self) -> str:
            return next(self.inputs)

        def print_reply(self, message: str) -> None:
            self.pieces.append(("reply", message))

        def print_reply_piece(self, piece: str) -> None:
            self.pieces.append(("piece", piece))

    view = View()
    bot = StandardChatbot(gen, enc, tok.create_decoder(skip_special_tokens=True))
    ChatbotProgram(view, bot, gen, tok, FakeGang(device=dev), enc).run()
    assert ("reply", "Bye!\n") in view.pieces and ("piece", "\n") in view.pieces


def _write_speech_data(root: Path, n: int = 12) -> Path:
    import struct

    audio = root / "audio"
    audio.mkdir(parents=True)
    man = root / "manifest"
    man.mkdir()
    g = torch.Generator().manual_seed(0)
    for split, count in (("train", n), ("valid", 4)):
        rows, texts = [], []
        for i in range(count):
            num = 3000 + 250 * i
            t = torch.arange(num) / 16000
            wav = (0.3 * torch.sin(2 * torch.pi * (200 + 40 * i) * t) + 0.05 * torch.randn(num, generator=g))
            pcm = (wav.clamp(-1, 1) * 32767).to(torch.int16).numpy().tobytes()
            name = f"{split}_{i}.wav"
            with open(audio / name, "wb") as fp:
                fp.write(b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " +
                         struct.pack("<IHHIIHH", 16, 1, 1, 16000, 32000, 2, 16) + b"data" +
                         struct.pack("<I", len(pcm)) + pcm)
            rows.append(f"{name}\t{num}")
            texts.append("ab ba"[: 3 + i % 3])
        (man / f"{split}.tsv").write_text(str(audio) + "\n" + "\n".join(rows) + "\n")
        (man / f"{split}.wrd").write_text("\n".join(texts) + "\n")
    return man


def test_wav2vec2_ssl_and_asr_recipes(tmp_path: Path) -> None:
    from recipes.wav2vec2.asr.recipe import Wav2Vec2AsrRecipe
    from recipes.wav2vec2.ssl.recipe import Wav2Vec2SslRecipe

    man = _write_speech_data(tmp_path)
    common = ["--no-sweep-dir", "--no-exit-on-error", "--config", "model.arch=tiny",
              f"dataset.config_overrides={{path: {man}}}", "dataset.min_audio_len=1000", "dataset.max_audio_len=8000",
              "dataset.max_num_elements=16000", "dataset.npc=1", "trainer.mixed_precision.mode=off",
              "regime.num_steps=3", "regime.validate_every_n_steps=3", "regime.checkpoint_every_n_steps=3",
              "regime.publish_metrics_every_n_steps=1", "common.metric_recorders.jsonl=true"]
    out = tmp_path / "ssl"
    assert main(Wav2Vec2SslRecipe(), [str(out), *common, "lr_scheduler.config.num_warmup_steps=1",
                                      "optimizer.config.lr=1e-4"]) == 0
    rows = [json.loads(l) for l in open(out / "metrics" / "train.jsonl")]
    assert len(rows) == 3
    assert (out / "metrics" / "valid.jsonl").exists() and (out / "checkpoints" / "step_3").is_dir()

    out = tmp_path / "asr"
    assert main(Wav2Vec2AsrRecipe(), [str(out), *common, "tokenizer.name=char_tokenizer",
                                      "model.config_overrides={target_vocab_size: 300}",
                                      "trainer.freeze_encoder_for_n_steps=1", "regime.validate_after_n_steps=0"]) == 0
    valid = [json.loads(l) for l in open(out / "metrics" / "valid.jsonl")]
    assert valid and any("wer" in k.lower() for k in valid[-1])


def test_lm_dpo_recipe(tmp_path: Path) -> None:
    from recipes.lm.dpo.recipe import LMDPORecipe

    data = tmp_path / "pref.jsonl"
    with open(data, "w") as fp:
        for i in range(32):
            fp.write(json.dumps({"src": f"Is {i} even? ", "tgt_chosen": "yes" if i % 2 == 0 else "no",
                                 "tgt_rejected": "no" if i % 2 == 0 else "yes"}) + "\n")
    args = [str(tmp_path / "out"), "--no-sweep-dir", "--no-exit-on-error", "--config", "model.name=null",
            "model.family=llama", "model.arch=tiny", "reference_model.name=null", "reference_model.family=llama",
            "reference_model.arch=tiny", "reference_model.dtype=float32", "tokenizer.name=char_tokenizer",
            f"dataset.config_overrides={{path: {data}}}", "dataset.batch_size=4", "dataset.max_seq_len=64",
            "trainer.mixed_precision.mode=off", "optimizer.config.lr=1e-4", "lr_scheduler.config.num_warmup_steps=1",
            "criterion.beta=0.5", "criterion.nll_scale=0.1", "regime.num_steps=4",
            "regime.checkpoint_every_n_steps=4", "regime.publish_metrics_every_n_steps=1",
            "common.metric_recorders.jsonl=true"]
    assert main(LMDPORecipe(), args) == 0
    rows = [json.loads(l) for l in open(tmp_path / "out" / "metrics" / "train.jsonl")]
    assert len(rows) == 4 and all(math.isfinite(r["dpo_loss"]) for r in rows)


def _tp_sft_worker(rank: int, world: int, root: str, seq_par: bool):
    from recipes.lm.sft.recipe import LMSFTRecipe

    tmp = Path(root)
    data = tmp / "data"
    args = _sft_args(tmp, data, ["regime.num_steps=3", "dataset.packed=true", "gang.tensor_parallel_size=2",
                                 f"gang.sequence_parallel={str(seq_par).lower()}", "trainer.data_parallelism=fsdp",
                                 "regime.validate_every_n_steps=null", "regime.checkpoint_every_n_steps=null"])
    return main(LMSFTRecipe(), args)


@pytest.mark.parametrize("seq_par", [True, False])
def test_lm_sft_recipe_with_tensor_parallelism(tmp_path: Path, seq_par: bool) -> None:
    """Two gloo ranks, TP=2: the recipe builds the LLaMA model sequence parallel (token-sharded residual stream,
    vocabulary-parallel embedding and loss) or with replicated activations, and the loss goes down either way."""
    from tests.dist_utils import run_distributed

    _write_sft_data(tmp_path)
    assert run_distributed(_tp_sft_worker, 2, str(tmp_path), seq_par, timeout=300.0) == [0, 0]
    lines = [json.loads(l) for l in open(tmp_path / "out" / "metrics" / "train.jsonl")]
    assert len(lines) == 3 and lines[-1]["NLL Loss"] < lines[0]["NLL Loss"]


def _pretrained_sft_worker(rank: int, world: int, root: str, ckpt: str):
    from recipes.lm.sft.recipe import LMSFTRecipe

    tmp = Path(root)
    args = _sft_args(tmp, tmp / "data", ["regime.num_steps=2", "dataset.packed=true", "trainer.data_parallelism=fsdp",
                                         f"model.path={ckpt}", "optimizer.config.lr=1e-6",
                                         "regime.validate_every_n_steps=null", "regime.checkpoint_every_n_steps=null"])
    return main(LMSFTRecipe(), args)


def test_lm_sft_recipe_fine_tunes_pretrained_weights_on_two_fsdp_ranks(tmp_path: Path) -> None:
    """`model.path` points at a consolidated checkpoint; the job runs on two ranks with FSDP. The model is loaded
    whole and sharded afterwards, and the first loss is the pretrained model's, not a fresh one's."""
    import torch

    from fairseq2_b200.models.family import get_model_family
    from tests.dist_utils import run_distributed

    _write_sft_data(tmp_path)
    fam = get_model_family("llama")
    cfg = fam.get_arch_config("tiny")
    torch.manual_seed(1)
    model = fam.create_new_model(cfg, None)
    with torch.no_grad():
        # "pretrained" in a way the loss can tell: the output projection is zero, so every token is equally likely
        model.final_proj.weight.zero_()
    ckpt = tmp_path / "pretrained.pt"
    torch.save({"model": model.state_dict()}, ckpt)
    assert run_distributed(_pretrained_sft_worker, 2, str(tmp_path), str(ckpt), timeout=300.0) == [0, 0]
    lines = [json.loads(l) for l in open(tmp_path / "out" / "metrics" / "train.jsonl")]
    uniform = math.log2(cfg.vocab_size)                   # the metric is in bits
    assert abs(lines[0]["NLL Loss"] - uniform) < 1e-2 * uniform, (lines[0]["NLL Loss"], uniform)


def _continue_worker(rank: int, world: int, root: str, prev: str):
    from recipes.lm.sft.recipe import LMSFTRecipe

    tmp = Path(root)
    args = _sft_args(tmp, Path(prev) / "data", [
        "regime.num_steps=2", "dataset.packed=true", "trainer.data_parallelism=fsdp", "model.name=last_checkpoint",
        "model.family=null", "model.arch=null", f"common.assets.prev_checkpoint_dir={prev}/out/checkpoints",
        "optimizer.config.lr=1e-6", "regime.validate_every_n_steps=null", "regime.checkpoint_every_n_steps=null"])
    return main(LMSFTRecipe(), args)


def test_checkpoint_of_one_run_is_the_model_asset_of_the_next_at_another_world_size(tmp_path: Path) -> None:
    """A run on one process writes checkpoints; a second job on two FSDP ranks names `last_checkpoint` of that
    directory as its model and starts from the trained weights (its first loss is near the first run's last)."""
    from recipes.lm.sft.recipe import LMSFTRecipe
    from tests.dist_utils import run_distributed

    first_dir, second_dir = tmp_path / "first", tmp_path / "second"
    first_dir.mkdir(), second_dir.mkdir()
    data = _write_sft_data(first_dir)
    assert main(LMSFTRecipe(), _sft_args(first_dir, data, ["regime.num_steps=4", "dataset.packed=true"])) == 0
    first = [json.loads(l) for l in open(first_dir / "out" / "metrics" / "train.jsonl")]
    assert run_distributed(_continue_worker, 2, str(second_dir), str(first_dir), timeout=300.0) == [0, 0]
    second = [json.loads(l) for l in open(second_dir / "out" / "metrics" / "train.jsonl")]
    assert first[0]["NLL Loss"] > 10 and second[0]["NLL Loss"] < first[-1]["NLL Loss"] + 1.0


def _resume_worker(rank: int, world: int, root: str, steps: int):
    from recipes.lm.sft.recipe import LMSFTRecipe

    tmp = Path(root)
    args = _sft_args(tmp, tmp / "data", [
        f"regime.num_steps={steps}", "dataset.packed=true", "trainer.data_parallelism=fsdp",
        "lr_scheduler.config.cycle_len=8",                 # the schedule must not depend on where a run stops
        "regime.validate_every_n_steps=null", "regime.checkpoint_every_n_steps=2"])
    return main(LMSFTRecipe(), args)


def test_two_rank_fsdp_run_resumes_where_it_stopped(tmp_path: Path) -> None:
    """Four steps on two FSDP ranks, then the same command with six: the second job restores model, optimizer,
    trainer and data position from the checkpoint of step 4 -- which here falls exactly on the end of the first data
    epoch -- and its steps 5 and 6 equal those of a job that ran six steps in one go."""
    from tests.dist_utils import run_distributed

    once, twice = tmp_path / "once", tmp_path / "twice"
    once.mkdir(), twice.mkdir()
    _write_sft_data(once), _write_sft_data(twice)
    assert run_distributed(_resume_worker, 2, str(once), 6, timeout=300.0) == [0, 0]
    assert run_distributed(_resume_worker, 2, str(twice), 4, timeout=300.0) == [0, 0]
    assert run_distributed(_resume_worker, 2, str(twice), 6, timeout=300.0) == [0, 0]
    want = [json.loads(l)["NLL Loss"] for l in open(once / "out" / "metrics" / "train.jsonl")]
    got = [json.loads(l)["NLL Loss"] for l in open(twice / "out" / "metrics" / "train.jsonl")]
    assert len(want) == 6 and len(got) == 6
    assert got == pytest.approx(want, rel=1e-4)


def _ssl_layerdrop_worker(rank: int, world: int, root: str, man: str, data_parallelism: str):
    from recipes.wav2vec2.ssl.recipe import Wav2Vec2SslRecipe

    args = [str(Path(root) / "ssl"), "--no-sweep-dir", "--no-exit-on-error", "--config", "model.arch=tiny",
            "model.config_overrides={encoder_config: {layer_drop_p: 0.5}}", f"dataset.config_overrides={{path: {man}}}",
            "dataset.min_audio_len=1000", "dataset.max_audio_len=8000", "dataset.max_num_elements=16000", "dataset.npc=1",
            "trainer.mixed_precision.mode=off", f"trainer.data_parallelism={data_parallelism}", "regime.num_steps=4",
            "regime.validate_every_n_steps=null", "regime.checkpoint_every_n_steps=null",
            "regime.publish_metrics_every_n_steps=1", "common.metric_recorders.jsonl=true",
            "lr_scheduler.config.num_warmup_steps=1", "optimizer.config.lr=1e-4"]
    return main(Wav2Vec2SslRecipe(), args)


@pytest.mark.parametrize("data_parallelism", ["ddp", "fsdp"])
def test_wav2vec2_ssl_with_layer_drop_on_two_ranks(tmp_path: Path, data_parallelism: str) -> None:
    """LayerDrop really skips layers. Jobs seed every rank differently, so two ranks would drop different layers:
    fine for replicated parameters (missing gradients count as zero), but with sharded units over process-group
    collectives every rank has to run the same layers -- the engine then makes the decisions identical."""
    from tests.dist_utils import run_distributed

    man = _write_speech_data(tmp_path)
    assert run_distributed(_ssl_layerdrop_worker, 2, str(tmp_path), str(man), data_parallelism, timeout=240.0) == [0, 0]
    rows = [json.loads(l) for l in open(tmp_path / "ssl" / "metrics" / "train.jsonl")]
    assert len(rows) == 4

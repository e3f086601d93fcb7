"""The end-to-end example on CPU: data and model preparation scripts, the Hugging Face checkpoint layout, and
examples/train_ddp.py with two ranks on the backend's host executor against the same run on gloo."""
import json
import os
import re
import socket
import subprocess
import sys

import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(cmd, cwd, timeout=600):
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(cmd, cwd=cwd, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def test_synthetic_records_and_dataset(tmp_path):
    from stragglar_b200.utils.data import (ByteTokenizer, InstructionDataset, format_example, load_records, save_records,
                                           synthetic_records)
    recs = synthetic_records(32, seed=3)
    assert recs == synthetic_records(32, seed=3) and recs != synthetic_records(32, seed=4)
    save_records(recs, str(tmp_path / "d"))
    assert load_records(str(tmp_path / "d")) == recs
    assert len(load_records(str(tmp_path / "d"), limit=5)) == 5
    text = format_example({"instruction": "Add.", "input": "1 2", "output": "3"})
    assert text == "### Instruction:\nAdd.\n\n### Input:\n1 2\n\n### Response:\n3"
    assert "### Input" not in format_example({"instruction": "Hi.", "input": "", "output": "x"})
    tok = ByteTokenizer()
    assert tok.decode(tok.encode("héllo")) == "héllo"
    ds = InstructionDataset(recs, tok, max_length=48)
    item = ds[0]
    assert item["input_ids"].shape == (48,) and item["input_ids"][0] == tok.bos_id
    pad = item["attention_mask"] == 0
    assert (item["labels"][pad] == -100).all() and (item["labels"][~pad] == item["input_ids"][~pad]).all()
    with pytest.raises(FileNotFoundError):
        load_records(str(tmp_path / "missing"))


def test_checkpoint_roundtrip_and_rope_scaling(tmp_path):
    from stragglar_b200.models import LlamaConfig, LlamaForCausalLM
    from stragglar_b200.models.llama import rope_tables
    cfg = LlamaConfig.tiny()
    cfg.rope_scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    cfg.tie_embeddings = False
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg)
    m.save_pretrained(str(tmp_path / "ck"))
    hf_cfg = json.load(open(tmp_path / "ck" / "config.json"))
    assert hf_cfg["num_key_value_heads"] == cfg.num_kv_heads and hf_cfg["rope_scaling"]["rope_type"] == "llama3"
    m2 = LlamaForCausalLM.from_pretrained(str(tmp_path / "ck"))
    ids = torch.randint(0, cfg.vocab_size, (2, 24))
    assert torch.equal(m(ids), m2(ids))
    # scaling stretches the long wavelengths only
    c0, _ = rope_tables(16, cfg.head_dim, 100.0, "cpu")
    c1, _ = rope_tables(16, cfg.head_dim, 100.0, "cpu", scaling=cfg.rope_scaling)
    assert torch.equal(c0[:, 0], c1[:, 0]) and not torch.equal(c0[:, -1], c1[:, -1])
    # a checkpoint of another shape is refused
    deeper = LlamaConfig.tiny()
    deeper.num_layers = 3
    other = LlamaForCausalLM(deeper)
    with pytest.raises((KeyError, RuntimeError)):
        other.load_hf_state_dict(m.hf_state_dict())


def test_model_matches_transformers_llama(tmp_path):
    transformers = pytest.importorskip("transformers")
    from stragglar_b200.models import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig.tiny()
    cfg.rope_scaling = {"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    torch.manual_seed(1)
    m = LlamaForCausalLM(cfg)
    m.save_pretrained(str(tmp_path / "ck"))
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ck"), dtype=torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (2, 40))
    labels = ids.clone()
    labels[:, 30:] = -100
    with torch.no_grad():
        assert (m(ids) - hf(ids).logits).abs().max().item() < 1e-4
        assert abs(m(ids, labels=labels).item() - hf(ids, labels=labels).loss.item()) < 1e-4


def _losses(out: str):
    got = {}
    for rank, step, loss in re.findall(r"Rank (\d+) \| Step (\d+) \|.*?Loss: ([0-9.]+)", out):
        got[(int(rank), int(step))] = float(loss)
    return got


def test_train_ddp_script_on_cpu_matches_gloo(tmp_path):
    cwd = str(tmp_path)
    out = _run([sys.executable, os.path.join(REPO, "examples", "load_dataset.py"), "--samples", "48"], cwd)
    assert "48 synthetic records" in out
    _run([sys.executable, os.path.join(REPO, "examples", "load_model.py"), "--tiny", "--dtype", "float32", "--out", "tiny"], cwd)
    runs = {}
    for backend in ("stragglar", "nccl"):   # with --cpu the stock arm is gloo
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), os.path.join(REPO, "examples", "train_ddp.py"), "--cpu",
               "--backend", backend, "--model-dir", "tiny", "--data-dir", "alpaca", "--max-length", "48", "--micro-batch",
               "2", "--steps", "3", "--warmup", "1", "--dtype", "float32", "--delay-ms", "1"]
        out = _run(cmd, cwd)
        assert re.search(rf"RESULT backend={backend} .*world=2 .*tokens_per_s=\d+", out), out[-2000:]
        runs[backend] = _losses(out)
    assert len(runs["stragglar"]) == 8 and runs["stragglar"].keys() == runs["nccl"].keys()
    for k, v in runs["stragglar"].items():
        assert abs(v - runs["nccl"][k]) < 2e-3, (k, v, runs["nccl"][k])
    # training moves the loss
    assert runs["stragglar"][(0, 3)] != runs["stragglar"][(0, 0)]

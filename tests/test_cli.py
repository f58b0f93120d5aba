"""The command line: the parts that need no GPU, and generation on the GPU."""
import json
import os
import subprocess
import sys

import pytest

import harness as H
from tiny_configs import TINY_A

from lastengine_b200.cli import build_parser, main, parse_ids

EXE = os.path.join(H.ROOT, "bin", "lastengine")


def test_prompt_ids_and_reference_flag_names():
    assert parse_ids("1, 5,17") == [1, 5, 17] and parse_ids("3 4") == [3, 4]
    with pytest.raises(SystemExit):
        parse_ids("hello")
    a = build_parser().parse_args(["generate", "--model", "m", "--prompt-ids", "1,2", "--temperature", "0.8", "--top-k", "40",
                                   "--top-p", "0.9", "--min-p", "0.1", "--presence-penalty", "0.5", "--repeat-penalty", "1.1",
                                   "--seed", "7", "--ctx", "512"])
    assert (a.temperature, a.top_k, a.top_p, a.min_p, a.presence_penalty, a.repeat_penalty, a.seed, a.ctx) == \
        (0.8, 40, 0.9, 0.1, 0.5, 1.1, 7, 512)
    d = build_parser().parse_args(["generate", "--model", "m", "--prompt-ids", "1"])
    assert (d.temperature, d.top_p, d.top_k, d.min_p, d.repeat_penalty) == (0.7, 0.95, 40, 0.0, 1.0)   # the reference's defaults
    g = build_parser().parse_args(["gpu", "dir", "1,2,3"])
    assert g.top == 5 and build_parser().parse_args(["tf-dump", "dir", "1"]).n == 100


def test_init_and_inspect(tmp_path, capsys):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    assert main(["init", "--config", str(cfg), "--seed", "3", "--out", str(out)]) == 0
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    capsys.readouterr()
    assert main(["inspect", str(out)]) == 0
    text = capsys.readouterr().out
    assert "4 layers" in text and "layer 1: attention + swiglu" in text and "173056 parameters" in text
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps(dict(TINY_A, architectures=["Nope"])))
    assert main(["inspect", str(bad)]) == 1
    assert "unknown architecture 'Nope'" in capsys.readouterr().err


@pytest.mark.gpu
def test_generate_gpu_and_tf_dump(tmp_path):
    d = H.make_model_dir(TINY_A, 0, str(tmp_path / "m"))
    p = subprocess.run([sys.executable, EXE, "generate", "--model", d, "--dtype", "float32", "--prompt-ids", "1,2,3",
                        "--prompt-ids", "9 8 7 6 5", "--max-new-tokens", "5", "--temperature", "0", "--stop-token-id", "255"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-1500:]
    rows = [json.loads(l) for l in p.stdout.splitlines()]
    assert len(rows) == 2 and all(len(r["tokens"]) <= 5 for r in rows)
    p2 = subprocess.run([sys.executable, EXE, "tf-dump", d, "1,2,3", "5", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert p2.returncode == 0, p2.stderr[-1500:]
    dump = json.loads(p2.stdout.splitlines()[-1])
    assert dump["prompt_ids"] == [1, 2, 3] and len(dump["gen_ids"]) == 5 and len(dump["top"][0]) == 5
    if len(rows[0]["tokens"]) == 5:
        assert dump["gen_ids"] == rows[0]["tokens"]          # greedy both ways
    p3 = subprocess.run([sys.executable, EXE, "gpu", d, "1,2,3", "3", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert p3.returncode == 0 and p3.stdout.count("logprob") == 3 and "greedy:" in p3.stdout
    p5 = subprocess.run([sys.executable, EXE, "dense-cmp", d, "1,2,3", "6"], capture_output=True, text=True, timeout=600)
    assert p5.returncode == 0, p5.stderr[-1500:]
    last = p5.stdout.splitlines()[-1]
    assert last.endswith(tuple("0123456789")) and "/6 argmax agree, mean |dlogprob|" in last
    assert float(last.rsplit("max ", 1)[1]) < 0.05               # bfloat16 against the true 32-bit path
    p4 = subprocess.run([sys.executable, EXE, "probe", "--json"], capture_output=True, text=True, timeout=300)
    assert json.loads(p4.stdout)["gpus"][0]["sm_count"] > 0

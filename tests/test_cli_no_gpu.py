"""The command line's verbs that need no GPU (random, info, doctor), and what the others say
on a machine without one."""
import json

import pytest
import torch

from tiny_configs import TINY_B


def test_random_then_info(tmp_path, capsys):
    from mivi_v4_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_B))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--seed", "1", "--out", str(out)]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "architecture: Lfm2ForCausalLM" in text and "(ff_dim: 256)" in text
    assert "model.layers.0.self_attn.q_layernorm.weight" in text and "model.layers.1.conv.in_proj.bias" in text
    assert "lm_head.weight" in text                                   # TINY_B has an untied head


def test_doctor_reports_the_compiler_and_the_libraries(capsys):
    from mivi_v4_b200.cli import main
    assert main(["doctor"]) == 0
    text = capsys.readouterr().out
    assert "nvcc:" in text and "core:" in text and "bf16:" in text


@pytest.mark.skipif(torch.cuda.is_available(), reason="a GPU is there")
def test_gpu_verbs_refuse_clearly_without_a_gpu(tmp_path, capsys):
    from mivi_v4_b200.cli import main
    assert main(["generate", "-m", str(tmp_path), "--prompt-ids", "1,2"]) == 2
    err = capsys.readouterr().err
    assert "no CUDA device" in err and "Traceback" not in err


def test_the_librarys_own_errors_are_one_line(tmp_path, capsys):
    from mivi_v4_b200.cli import main
    assert main(["info", "-m", str(tmp_path / "nothing_here")]) == 1
    err = capsys.readouterr().err
    assert err.startswith("mivi info: ConfigError: no config.json") and "Traceback" not in err
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_B, num_hidden_layers=0)))
    assert main(["info", "-m", str(tmp_path)]) == 1
    assert "ConfigError" in capsys.readouterr().err

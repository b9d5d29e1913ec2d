"""What bench.py promises without a GPU: one line and exit status 2 for more than one GPU, the
reference arm's ``unavailable`` line, and where the roofline's denominators come from."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def run(*args, env=None):
    e = dict(os.environ)
    e.pop("WORLD_SIZE", None)
    e.update(env or {})
    p = subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, env=e, timeout=120)
    return p.returncode, [ln for ln in p.stdout.splitlines() if ln.strip()]


def test_more_than_one_gpu_is_refused_with_one_line():
    code, lines = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert code == 2 and len(lines) == 1
    assert "one GPU" in json.loads(lines[0])["error"]
    code, lines = run("--gpus", "1", env={"WORLD_SIZE": "4"})         # launched as one rank of several
    assert code == 2 and len(lines) == 1


def test_reference_arm_says_why_it_is_unavailable():
    code, lines = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert code == 0 and len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["unavailable"] and "\n" not in rec["unavailable"]


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    pk, src = bench.peaks()
    assert src == "fallback" and pk == bench.FALLBACK_PEAKS
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"hbm_gbs": 7001.5, "gemm": {"bf16_tflops": 1612, "bf16_tflops_sustained": 1433}, "note": "x", "sm_mhz": 1900}))
    pk, src = bench.peaks()
    assert src == "measured"
    assert pk == {"hbm_gbs": 7001.5, "bf16_tflops": 1612.0, "bf16_tflops_sustained": 1433.0}
    (tmp_path / "MEASURED_PEAKS.json").write_text("{ not json")
    assert bench.peaks()[1] == "fallback"


def test_benchmark_configuration_is_the_named_one():
    """The sizes of the benchmark's default run, as a configuration of the library."""
    sys.path.insert(0, ROOT)
    import bench
    from mivi_v4_b200.config import Lfm2Config
    c = Lfm2Config.from_dict(bench.BENCH_CONFIG)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (16, 2048, 32, 8)
    assert (c.head_dim, c.ff_dim, c.vocab_size, c.conv_L_cache) == (64, 8192, 65536, 3)
    assert list(c.attn_layer_ids) == [2, 5, 8, 10, 12, 14] and c.tie_embedding
    assert bench.CONTEXT == 4096 and bench.PROMPT == 512 and bench.PREFILL_TOKENS == 2048


def test_clock_record_prefers_the_denser_source(monkeypatch):
    """With NVML readable the clocks come from it (a sample every 20 ms); without, from nvidia-smi;
    with neither the record is empty, never an error."""
    import time
    import types

    import torch  # noqa: F401  (the sampler asks it for the GPU's UUID; a first import takes seconds)
    sys.path.insert(0, ROOT)
    import bench
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: "h"

    def by_uuid(u):
        raise RuntimeError("unknown")
    fake.nvmlDeviceGetHandleByUUID = by_uuid
    fake.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965
    clocks = iter([1965, 1950, 1900] + [1965] * 10000)
    fake.nvmlDeviceGetClockInfo = lambda h, k: next(clocks)
    fake.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: 0x4 | 0x1          # power cap, and "idle" (not kept)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    with bench.ClockSampler() as c:
        time.sleep(0.25)
    rec = c.summary()
    assert rec["source"] == "nvml" and rec["samples"] >= 5
    assert rec["sm_mhz"] == 1965.0 and rec["sm_max_mhz"] == 1965.0 and rec["reasons"] == ["sw_power_cap"]

    broken = types.ModuleType("pynvml")                                        # NVML that cannot start
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    with bench.ClockSampler() as c:
        time.sleep(0.05)
    rec = c.summary()
    assert rec["samples"] == 0 and rec["sm_mhz"] is None and rec["reasons"] == []

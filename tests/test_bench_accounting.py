"""The arithmetic behind bench.py's roofline figures: the flops of a prefill step and the peaks it divides by.  The
figures for the 1.5B shape are worked out by hand here (per layer: q|k|v 2 x 1536 x 2048, o 2 x 1536 x 1536, gate|up and
down 2 x 3 x 1536 x 8960 flops a token; causal attention 4 x 12 x 128 flops a (query, key) pair)."""

from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def test_prefill_flops_of_the_benchmark_shape():
    cfg = bench.bench_config()
    assert (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
            cfg["intermediate_size"], cfg["vocab_size"]) == (28, 1536, 12, 2, 128, 8960, 151936)
    T = 2048
    linear = 2 * T * 28 * (1536 * 2048 + 1536 * 1536 + 3 * 1536 * 8960)
    attention = 4 * 12 * 128 * (T * (T + 1) // 2) * 28
    head = 2 * 1536 * 151936                                       # one row of logits
    assert bench.decode_flops_and_prefill_flops(cfg, T) == linear + attention + head
    assert abs(bench.decode_flops_and_prefill_flops(cfg, T) / 1e12 - 5.73) < 0.01      # 5.37 linear + 0.36 attention


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    assert bench.load_peaks()["source"] == "fallback" and bench.load_peaks()["hbm_gbs"] == 6650.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 7012.5, "bf16_tflops": 1611.0, "bf16_tflops_sustained": 1402.0}))
    p = bench.load_peaks()
    assert (p["source"], p["hbm_gbs"], p["bf16_tflops"], p["bf16_tflops_sustained"]) == ("measured", 7012.5, 1611.0, 1402.0)
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert bench.load_peaks()["source"] == "fallback"


def test_more_than_one_gpu_is_refused_with_one_line(capsys, monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "2"])
    assert bench.main() == 2
    out = capsys.readouterr().out.strip().splitlines()
    assert len(out) == 1 and "one GPU" in out[0]
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference"])
    assert bench.main() == 0
    line = json.loads(capsys.readouterr().out)
    assert line["impl"] == "reference" and "unavailable" in line

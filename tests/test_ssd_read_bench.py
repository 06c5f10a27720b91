import os

from fastllm_b200.utils import ssd_read_bench


def test_read_bench_counts_bytes(tmp_path):
    for i in range(3):
        (tmp_path / f"w{i}.safetensors").write_bytes(os.urandom((i + 1) << 20))
    (tmp_path / "notes.txt").write_text("ignored")
    r = ssd_read_bench.read_bench([str(tmp_path)], threads=3, seconds=0.3, block_mb=1)
    assert r["files"] == 3 and r["reads"] > 0 and r["bytes"] == r["reads"] << 20 and r["gb_per_s"] > 0

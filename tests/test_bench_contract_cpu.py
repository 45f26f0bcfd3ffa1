"""The reference arm of bench.py runs on the host alone (the CPU oracle of the BERT-base layer on a bounded
sample): check that it prints one JSON line with the keys the benchmark contract asks for."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "bert_base_layer_seqs_per_sec" and d["unit"] == "seq/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["steps"] == 1
    assert d["config"]["workload"].startswith("BERT-base encoder layer")
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "sample" in cb
    e2e = d["e2e"]
    assert e2e["value"] == d["value"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_ops_suite_cases_are_labelled_and_filterable():
    """`bench.py --suite ops --only <text>` selects cases by label `<config>:<op>:<shape>`; building the case list
    touches no GPU, the labels are unique, and every benchmark configuration has its rows."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from aitemplate_b200.testing import benchmark_ops

    labels = [label for label, _ in benchmark_ops._suite_cases({}, 1e12)]
    assert len(labels) == len(set(labels))
    for config in "12345":
        assert any(label.startswith(config + ":") for label in labels)
    assert "5:gemm:16x8192x8192" in labels and "2:attention:64x12x384x384x64" in labels
    assert [label for label in labels if "5:gemm:16x" in label] == ["5:gemm:16x8192x8192"]

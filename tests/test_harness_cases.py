"""The latency harness: its workload list mirrors benchmarks/moba_compare.py:59-99, which
yields 40 distinct shapes after its own de-duplication, every one of them inside what the
library accepts (checked without a GPU); one small case measured end to end on the GPU."""
import pytest

from baselinebenchmark_b200 import harness
from baselinebenchmark_b200.parallel import HEAD_DIMS


def test_suite_has_the_reference_case_count():
    cases = harness.reference_suite()
    assert len(cases) == 40
    assert len({c.name for c in cases}) == 40
    keys = {(c.seq_lens, c.q_heads, c.kv_heads, c.head_dim, c.chunk_size, c.topk, c.dtype) for c in cases}
    assert len(keys) == 40


def test_every_suite_case_is_supported():
    for case in harness.reference_suite():
        assert harness.supported(case), case
        assert case.head_dim in HEAD_DIMS
        assert case.q_heads % case.kv_heads == 0
        assert 1 <= case.topk <= 64


def test_baseline_cases_match_their_names():
    assert set(harness.BASELINE_CASES) == {"cfg0", "cfg1", "cfg2", "cfg3-unit", "cfg3-seq"}
    cfg2 = harness.BASELINE_CASES["cfg2"]
    assert (cfg2.seq_lens, cfg2.q_heads, cfg2.kv_heads, cfg2.chunk_size, cfg2.topk) == ((32768,), 32, 8, 4096, 12)


def test_summary_reports_p99_only_with_enough_samples():
    few = harness.summary([1.0, 2.0, 3.0])
    assert "p99_ms" not in few and few["median_ms"] == 2.0 and few["count"] == 3
    many = harness.summary([float(i) for i in range(200)])
    assert many["p99_ms"] == 197.0


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--backward"], ["--stage", "gating"]], ids=["forward", "backward", "gating"])
def test_harness_measures_a_baseline_case(extra, tmp_path):
    """The harness end to end on BASELINE.json configs[0]: one measured case with a latency
    summary, written as JSON (forward, --backward and the gating stage alone)."""
    import json
    out = tmp_path / "report.json"
    report = harness.main(["--case", "cfg0", "--rounds", "1", "--iterations", "2", "--warmup", "1",
                           "--output", str(out)] + extra)
    (case,) = report["cases"]
    assert case["status"] == "measured" and case["latency"]["count"] == 2 and case["latency"]["median_ms"] > 0
    assert json.loads(out.read_text())["cases"][0]["name"] == "cfg0"

"""The static rules for CUDA sources: the tree is clean, and each rule fires on a minimal offending snippet."""
from opaque_b200.utils import source_rules as R

MC = "multicast" + "::" + "cluster"
BATCH = "cudaMemcpy" + "Batch" + "Async"


def _rules(path, text):
    return sorted({f.rule for f in R.check_text(path, text)})


def test_repository_sources_are_clean():
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    found = R.check_tree(root)
    assert not found, "\n".join(map(str, found))


def test_each_rule_fires():
    assert _rules("k.cu", 'asm volatile("mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;");') == ["raw-mbarrier-wait"]
    helper = '__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {\n  asm volatile("mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;");\n}\n'
    assert _rules("csrc/common.cuh", helper) == [] and _rules("csrc/other.cuh", helper) == ["raw-mbarrier-wait"]
    assert _rules("k.cu", f'asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.{MC} [%0], [%1, {{%2, %3}}], [%4], %5;");') == ["multicast-load"]
    assert _rules("k.cu", f'asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.{MC}.b64 [%0], %1;");') == []
    assert _rules("k.cu", "  if (bad) __trap();") == ["device-trap"] and _rules("k.cu", "  assert(i < n);") == ["device-trap"]
    assert _rules("k.cu", "static_assert(sizeof(int) == 4, \"int\");") == []
    assert _rules("a.py", f"lib.{BATCH}(ptrs)") == ["batched-copy-api"] and _rules("k.cu", f"  {BATCH}(a, b);") == ["batched-copy-api"]
    spin = "  while (*reinterpret_cast<volatile int*>(flag) < epoch) {\n  }\n"
    assert _rules("k.cu", spin) == ["unbounded-spin"]
    bounded = ("  while (*reinterpret_cast<volatile int*>(flag) < epoch) {\n"
               "    if (++tries > budget) { *status = 3; return; }\n  }\n")
    assert _rules("k.cu", bounded) == []
    assert _rules("k.cu", "  // while (volatile) in a comment\n  for (int i = 0; i < n; ++i) { x[i] = 0; }\n") == []


def test_command_line_reports_and_returns_nonzero(tmp_path, capsys):
    (tmp_path / "bad.cu").write_text("__global__ void k(int* f) {\n  while (*(volatile int*)f == 0) {\n  }\n}\n")
    assert R.main([str(tmp_path)]) == 1
    out = capsys.readouterr().out
    assert "bad.cu:2: [unbounded-spin]" in out and "1 finding(s)" in out
    (tmp_path / "bad.cu").write_text("__global__ void k(int* f) { f[0] = 1; }\n")
    assert R.main([str(tmp_path)]) == 0

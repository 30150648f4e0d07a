"""Host side without a GPU: the library loads and exports what include/hb200.h declares, the tune
keys behave as the reference's Tune::apply (src/metal/qwen.rs:296-389), the check rule, and the
loud failure when no device is present."""
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "hb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(hb200):
    import ctypes

    L = hb200.lib()
    names = declared_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/hb200.h but not exported"
    assert sorted(hb200.EXPORTS) == names
    assert isinstance(L, ctypes.CDLL)


def test_no_device_is_an_error_not_a_fallback(hb200):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(hb200.HbError) as e:
        hb200.Context(0)
    assert e.value.status == hb200.BACKEND and "no CPU path" in e.value.message


def test_tune_defaults_and_summary(hb200):
    t = hb200.Tune()
    assert t.get("prefill.block") == 2048 and t.get("gemm.tn") == 64 and t.get("gemm.mma") == 1 and t.get("gemm.auto") == 1
    assert t.get("moe.tile") == 16 and t.get("pf.fswi") == 2 and t.get("mv.auto") == 1 and t.get("mv.cold") == 1
    assert t.gemm_timed()
    s = t.summary()
    assert s.startswith("prefill.block=2048 rec.chunk=4 ") and " gemm.auto=1 gemm.mma=1 gemm.tn=64 gemm.mform=0 " in s
    assert " mv.persist=0 mv.persists=[] dec.sdpa=32 " in s and s.endswith("dn.tscale=0")


def test_tune_naming_a_kernel_turns_timing_off(hb200):
    for setting in ("gemm.mma=2", "gemm.tn=32", "gemm.mform=3"):
        t = hb200.Tune(setting)
        assert not t.gemm_timed() and " gemm.auto=0 " in t.summary(), setting
    t = hb200.Tune("gemm.auto=0")
    assert not t.gemm_timed()
    t = hb200.Tune("prefill.block=512,gemm.mfirst=0")
    assert t.gemm_timed() and t.get("prefill.block") == 512 and t.get("gemm.mfirst") == 0
    assert hb200.Tune("prefill.block=0").get("prefill.block") == 1
    assert hb200.Tune("mv.split=2").get("mv.auto") == 0 and hb200.Tune("mv.persist=1").get("mv.auto") == 0
    assert hb200.Tune("dec.sdpa=99").get("dec.sdpa") == 64
    t = hb200.Tune("mv.persists=2/4")
    assert " mv.persists=[2, 4] " in t.summary()


@pytest.mark.parametrize(
    "setting,message",
    [
        ("foo.bar=1", "--tune foo.bar: unknown"),
        ("gemm.tn", "--tune gemm.tn: key=value"),
        ("gemm.tn=x", "--tune gemm.tn=x: invalid digit found in string"),
        ("gemm.tn=", "--tune gemm.tn=: cannot parse integer from empty string"),
        ("gemm.tn=-1", "--tune gemm.tn=-1: invalid digit found in string"),
        ("gemm.tn=99999999999", "--tune gemm.tn=99999999999: number too large to fit in target type"),
        ("gemm.tn=48", "--tune gemm.mma=1 gemm.tn=48 gemm.mform=0: gemm.mma 0..2, gemm.tn 16, 32 or 64, gemm.mform 0..9"),
        ("gemm.mma=4", "--tune gemm.mma=4 gemm.tn=64 gemm.mform=0: gemm.mma 0..2, gemm.tn 16, 32 or 64, gemm.mform 0..9"),
        ("gemm.mform=10", "--tune gemm.mma=1 gemm.tn=64 gemm.mform=10: gemm.mma 0..2, gemm.tn 16, 32 or 64, gemm.mform 0..9"),
        ("moe.tile=48", "--tune moe.tile=48: 16, 32 or 64"),
        ("q4.fuse=2", "--tune q4.fuse=2: 0, or 1 with gemm.mma=1"),
    ],
)
def test_tune_errors_match_the_reference(hb200, setting, message):
    with pytest.raises(hb200.HbError) as e:
        hb200.Tune(setting)
    assert e.value.status == hb200.INVALID and e.value.message == message


def test_tune_failed_apply_changes_nothing(hb200):
    t = hb200.Tune("gemm.tn=32")
    with pytest.raises(hb200.HbError):
        t.apply("prefill.block=256,nope=1")
    assert t.get("prefill.block") == 2048 and t.get("gemm.tn") == 32
    assert hb200.Tune("gemm.mma=3,gemm.tn=128").get("gemm.tn") == 128  # 128 columns only with gemm.mma=3


def test_check_rule_matches_oracle(hb200, oracle):
    rng = np.random.default_rng(0)
    ref = rng.standard_normal(4096).astype(np.float32)
    for eps in (0.0, 0.9, 1.1, 5.0):
        got = ref.copy()
        got[100] += np.abs(ref).max() / 64 * eps
        a = hb200.check_rule(ref, got)
        b = oracle.check_1_64(ref, got)
        assert a[0] == b[0] and a[1] == pytest.approx(b[1]) and a[2] == pytest.approx(b[2])
    got = ref.copy()
    got[5] = np.nan
    assert hb200.check_rule(ref, got)[0] is False
    r16 = oracle.normal(1000, 1, 1, 1.0)
    g16 = r16.copy()
    assert hb200.check_rule(r16, g16)[0] is True
    g16[7] ^= 0x4000
    assert hb200.check_rule(r16, g16)[0] == oracle.check_1_64(r16, g16)[0]


def test_moe_tiles_bound(hb200):
    # ceil(rows*top_k / bm) + experts, src/metal/prefill.rs:832
    L = hb200.lib()
    assert L.hb_moe_tiles(2048, 8, 256, 16) == 1280 and L.hb_moe_tiles(2048, 8, 256, 32) == 768 and L.hb_moe_tiles(2048, 8, 256, 64) == 512
    assert L.hb_moe_tiles(1, 1, 1, 16) == 2


def test_integration_stub_declares_every_export(hb200):
    """The Rust extern block of INTEGRATION.md is meant to be pasted as the -sys file: it must name every function
    the header declares (and nothing the library does not export)."""
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "INTEGRATION.md")).read()
    block = text[text.index('extern "C" {') : text.index("/// Status ->")]
    in_stub = set(re.findall(r"pub fn (hb_[a-z0-9_]+)\(", block))
    header = open(os.path.join(root, "include", "hb200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", header))
    assert declared == set(hb200.EXPORTS), sorted(declared ^ set(hb200.EXPORTS))
    assert in_stub == declared, sorted(in_stub ^ declared)
    # the descriptors field for field
    for struct, cls in (("hb_gemm_desc", hb200.GemmDesc), ("hb_matvec_desc", hb200.MatvecDesc)):
        body = header[: header.index("} " + struct + ";")]
        body = body[body.rindex("typedef struct {") :]
        fields = re.findall(r"uint32_t\s+([a-z_0-9, ]+);", body)
        names = [n.strip() for f in fields for n in f.split(",")]
        assert names == [n for n, _ in cls._fields_], (struct, names)
        rust = re.search(r"pub struct " + struct + r" \{(.*?)\}", text, flags=re.S).group(1)
        assert re.findall(r"pub ([a-z_0-9]+): u32", rust) == names, struct

import json
import os

import pytest
import torch


def test_hex_hash_time(native):
    u = native.utils
    blob = bytes(range(256))
    assert u.decode_hex(u.encode_hex(blob)) == blob
    assert u.encode_hex(b"\x00\xff\x10") == "00ff10"
    with pytest.raises(RuntimeError):
        u.decode_hex("abc")
    with pytest.raises(RuntimeError):
        u.decode_hex("zz")
    assert u.fnv1a("") == 14695981039346656037
    assert u.fnv1a("a") == 0xaf63dc4c8601ec8c
    t0 = u.now_nanos(); assert u.now_nanos() >= t0 > 1_600_000_000 * 10**9
    assert len(u.launch_timestamp().split("-")) == 3


def test_env_registry(native):
    L = native.utils.LaunchEnvironments
    opts = L.listOpt()
    for name in ("PCCL_LOG_LEVEL", "PCCL_WORKSPACE_MB", "PCCL_SPIN_LIMIT", "PCCL_TRANSPORT", "PCCL_IB_DEVICE"):
        assert name in opts
    assert L.getEnv("PCCL_SURELY_NOT_SET") == ""
    L.registerOpt("PCCL_TEST_OPTION", "made by a test")
    assert "PCCL_TEST_OPTION" in L.listOpt() and L.helpOf("PCCL_TEST_OPTION") == "made by a test"
    L.setOverride("PCCL_TEST_OPTION", "42")
    assert L.getEnv("PCCL_TEST_OPTION") == "42"
    assert L.getEnv("PATH") == os.environ["PATH"]


def test_json_and_logging(native):
    u = native.utils
    doc = {"a": [1, 2.5, True, None, "x\n\"y\""], "b": {"c": -7, "d": 1e-3}}
    assert json.loads(u.json_roundtrip(json.dumps(doc))) == doc
    with pytest.raises(RuntimeError):
        u.json_roundtrip("{\"a\": [1, 2}")
    before = u.log_count("error")
    u.log("error", "test message 123")
    assert u.log_count("error") == before + 1
    with open(u.log_path()) as f:
        assert "test message 123" in f.read()


def test_type_registry(native):
    u = native.utils
    a = u.register_type(3, "cpu"); b = u.register_type(3, "cuda")
    assert u.register_type(3, "cpu") == a and a != b
    assert "cuda" in u.type_names(3)
    u.set_compatible("cuda_interpreter", 1, "bf16")
    assert u.executors_for(1, "bf16") == ["cuda_interpreter"]


def test_cpu_number_formats(native):
    u = native.utils
    for v in (0.0, 1.0, -2.5, 3.140625, 1e-3, 65504.0, 448.0, -448.0, 0.015625):
        assert u.bf16_roundtrip(v) == torch.tensor(v).bfloat16().float().item()
        assert u.f16_roundtrip(v) == torch.tensor(v).half().float().item()
    if hasattr(torch, "float8_e4m3fn"):
        xs = torch.linspace(-500, 500, 4001).tolist() + [2 ** -9, 2 ** -10 * 1.5, 0.0019]
        for v in xs:
            want = torch.tensor(v).clamp(-448, 448).to(torch.float8_e4m3fn).float().item()
            assert u.e4m3_roundtrip(v) == want, v


@pytest.mark.parametrize("dtype,name", [(torch.float32, "f32"), (torch.bfloat16, "bf16"), (torch.float16, "f16"),
                                        (torch.int32, "i32"), (torch.float64, "f64")])
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_cpu_reduce(native, dtype, name, op):
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(1000, generator=g) * 10).to(dtype)
    b = (torch.randn(1000, generator=g) * 10).to(dtype)
    hi = torch.float64 if dtype == torch.float64 else torch.float32
    if dtype.is_floating_point:
        want = {"sum": a.to(hi) + b.to(hi), "max": torch.maximum(a.to(hi), b.to(hi)),
                "min": torch.minimum(a.to(hi), b.to(hi))}[op].to(dtype)
    else:
        want = {"sum": a + b, "max": torch.maximum(a, b), "min": torch.minimum(a, b)}[op]
    d = a.clone()
    assert native.utils.cpu_reduce(d.data_ptr(), b.data_ptr(), d.numel() * d.element_size(), name, op)
    assert torch.equal(d, want)

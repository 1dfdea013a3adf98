"""The C++ `Execution` class over stock libtorch (include/cswap_execution.hpp),
exercised by a small driver written like the reference's drivers
(tests/cpp/execution_driver.cpp)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_driver_lossless_policies_keep_gradients():
    from cswap_b200 import build
    exe = build.build_cpp_driver(name="execution_driver")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr[-2000:])
    assert r.returncode == 0 and "PASS" in r.stdout
    assert "policy 2:" in r.stdout and "policy 3:" in r.stdout and "policy 6:" in r.stdout


def test_cpp_vgg16_step_policies():
    """VGG16 at batch 128 under the C++ Execution (tests/cpp/vgg16_step.cpp --check):
    policies 1 / 2 / 3, the vDNN and SuperNeurons planners and the self-tuned
    lossless table are bit-identical to the step without swapping, the profile
    knows which activations nothing keeps, policy 6 hands backward exactly
    decode(encode(x)), and the engine's knobs (stream-ordered freeing, how far
    ahead tensors are brought back, staged payloads kept or not) leave the ZFP
    step's loss and gradients bit-identical."""
    from cswap_b200 import build
    exe = build.build_cpp_driver(name="vgg16_step")
    r = subprocess.run([exe, "--check"], capture_output=True, text=True, timeout=600)
    print(r.stdout, r.stderr[-2000:])
    assert r.returncode == 0 and "PASS" in r.stdout
    for tag in ("policy 2 (raw)", "policy 3 (sparse)", "policy 1 (drop)", "policy_ 3 (vDNN)", "policy_ 4 (SuperNeurons)",
                "self-tuned (lossless)", "policy 6 on id 2", "policy 6 on id 6", "blocks freed by polling",
                "three tensors ahead", "nothing kept staged", "nothing ahead"):
        assert tag in r.stdout


def test_cpp_vgg16_step_bench_line():
    import json
    from cswap_b200 import build
    exe = build.build_cpp_driver(name="vgg16_step")
    r = subprocess.run([exe, "--bench", "--steps", "3", "--warmup", "1"], capture_output=True, text=True, timeout=900)
    print(r.stderr[-2000:])
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    rows = d["rows"]
    assert {"no_swap", "raw_swap", "reference_split_zfp8", "zfp8_everywhere", "self_tuned"} <= set(rows)
    # raw copies of tensors that are taken back while they wait in the manager's queue are never made
    raw = rows["raw_swap"]
    assert rows["no_swap"]["link_bytes_out"] == 0 and 0 < raw["link_bytes_out"] <= raw["activation_bytes_swapped"]
    assert raw["activation_bytes_swapped"] > 2.5e8
    assert rows["zfp8_everywhere"]["link_bytes_out"] < 0.3 * raw["activation_bytes_swapped"]
    # a restored activation is freed as soon as its backward has used it: swapping lowers the peak
    assert rows["zfp8_everywhere"]["peak_device_mib"] < 0.9 * rows["no_swap"]["peak_device_mib"]
    h = d["hidden_activation_bytes"]
    assert set(h["per_policy"]) == {"raw", "compressed_reference_rule", "compressed_zfp8_everywhere"}


def test_cpp_bert_step_policies():
    """Two BERT-base-shaped layers (batch 32 x seq 512) under the C++ Execution
    (tests/cpp/bert_step.cpp --check): every activation swapped at its last
    forward use; raw and sparse leave loss and gradients bit-identical (same
    dropout seed), ZFP rate 16 leaves the loss identical and moves the gradients
    by a few per cent at most."""
    from cswap_b200 import build
    exe = build.build_cpp_driver(name="bert_step")
    r = subprocess.run([exe, "--check"], capture_output=True, text=True, timeout=900)
    print(r.stdout, r.stderr[-2000:])
    assert r.returncode == 0 and "PASS" in r.stdout
    for tag in ("policy 2:", "policy 3:", "policy 6:"):
        assert tag in r.stdout


def test_cpp_bert_step_bench_line():
    """The BERT-shaped step under the C++ Execution: ZFP rate 16 on every kept
    activation halves the link bytes and brings the peak of device memory well
    under the step without swapping."""
    import json
    from cswap_b200 import build
    exe = build.build_cpp_driver(name="bert_step")
    r = subprocess.run([exe, "--bench", "--layers", "4", "--steps", "2", "--warmup", "1"], capture_output=True, text=True,
                       timeout=900)
    print(r.stderr[-2000:])
    assert r.returncode == 0
    d = json.loads(r.stdout.strip().splitlines()[-1])
    rows = d["rows"]
    assert {"no_swap", "raw_swap", "zfp16_everywhere", "self_tuned"} <= set(rows)
    z, n = rows["zfp16_everywhere"], rows["no_swap"]
    assert z["swap_outs"] >= 10 * d["layers"] - 2 and z["taken_back"] == 0
    assert 0.45 * z["activation_bytes_swapped"] < z["link_bytes_out"] < 0.55 * z["activation_bytes_swapped"]
    assert z["peak_device_mib"] < 0.8 * n["peak_device_mib"]

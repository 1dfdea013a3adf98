"""Swap manager, cost model and the Execution mirror on a GPU."""
import numpy as np
import pytest

import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cs():
    import torch
    import cswap_b200
    assert torch.cuda.is_available()
    cswap_b200.lib()
    return cswap_b200


@pytest.fixture()
def mgr(cs):
    m = cs.SwapManager(pinned_bytes=256 << 20, staging_bytes=128 << 20)
    yield m
    m.close()


def test_raw_roundtrip(cs, mgr):
    import torch
    t = torch.from_numpy(util.normal(1 << 20, 1)).cuda()
    tk = mgr.swap_out(t, cs.POLICY_RAW)
    back = mgr.swap_in(tk)
    torch.cuda.synchronize()
    assert torch.equal(back, t)
    info = tk.info()
    assert info["policy"] == cs.POLICY_RAW and info["moved_bytes"] == 4 << 20 and info["complete"]
    tk.release()
    s = mgr.stats()
    assert s["swap_outs"] == 1 and s["swap_ins"] == 1 and s["pinned_in_use"] == 0 and s["staging_in_use"] == 0


def test_reclaim_before_departure_and_nonblocking_release(cs):
    """A losslessly swapped tensor that is wanted back while its copy out is
    still running is handed back as it is (no copy in); a lossy one never is;
    giving a ticket up while the device still reads its tensor does not block,
    and everything is returned to the pools once the copies have finished."""
    import time
    import torch
    m = cs.SwapManager(pinned_bytes=1 << 30, staging_bytes=256 << 20)
    big = torch.randn(64 << 20, device="cuda")       # 256 MiB: several ms on the host link
    keep = big.clone()
    torch.cuda.synchronize()
    tk = m.swap_out(big, cs.POLICY_RAW)
    back = m.reclaim(tk)
    assert back is big and m.reclaimed_tensors == 1   # the copy out cannot have finished yet
    assert m.reclaim(tk) is None                      # only once
    tz = m.swap_out(big, cs.POLICY_ZFP)
    assert m.reclaim(tz) is None                      # lossy: must come back decoded
    tr = m.swap_out(big, cs.POLICY_RAW)
    t0 = time.perf_counter()
    tr.release()                                      # still being read: parked, not waited for
    assert time.perf_counter() - t0 < 2e-3
    m.sync()
    torch.cuda.synchronize()
    assert torch.equal(big, keep)                     # the manager only ever read it
    dec = m.swap_in(tz)
    torch.cuda.synchronize()
    assert torch.equal(dec, cs.zfp_decompress(cs.zfp_compress(keep, 512), keep.numel(), 512))
    tz.release()
    done = m.swap_out(big, cs.POLICY_RAW)
    m.sync()
    assert m.reclaim(done) is None                    # it has left: a real swap-in is needed
    assert torch.equal(m.swap_in(done), keep)
    done.release()
    m.sync()
    s = m.stats()
    assert s["pinned_in_use"] == 0 and s["staging_in_use"] == 0 and not m._retiring and not m._reading
    m.close()


def test_blob_export_import_roundtrip(cs, tmp_path):
    """A swapped-out tensor written out as a self-describing blob and brought
    back through a different manager gives what swap_in of the original ticket
    would have given, for all three policies."""
    import numpy as np
    import torch
    a = cs.SwapManager(pinned_bytes=256 << 20, staging_bytes=128 << 20)
    b = cs.SwapManager(pinned_bytes=256 << 20, staging_bytes=128 << 20, zfp_maxbits=256)  # its own rate is irrelevant
    n = 3 * 1024 * 1024
    dense = torch.tanh(torch.randn(n, device="cuda"))
    relu = torch.relu(torch.randn(n, device="cuda") - 0.6)
    cases = [(cs.POLICY_RAW, dense, dense), (cs.POLICY_SPARSE, relu, relu),
             (cs.POLICY_ZFP, dense, cs.zfp_decompress(cs.zfp_compress(dense, 512), n, 512))]
    for pol, src, want in cases:
        tk = a.swap_out(src, pol)
        blob = tk.export()
        info = cs.blob_info(blob)
        assert info["policy"] == pol and info["numel"] == n and blob.size == 64 + info["payload_bytes"]
        assert info["zfp_maxbits"] == (512 if pol == cs.POLICY_ZFP else 0)
        if pol == cs.POLICY_SPARSE:
            assert info["nnz"] == int(torch.count_nonzero(relu).item())
        assert info["payload_bytes"] == tk.info()["moved_bytes"]
        tk.release()
        path = tmp_path / f"t{pol}.cswp"
        blob.tofile(path)                                     # outlives the ticket and the manager that made it
        tk2 = b.import_blob(np.fromfile(path, dtype=np.uint8), shape=(3, 1024, 1024))
        back = b.swap_in(tk2)
        torch.cuda.synchronize()
        assert back.shape == (3, 1024, 1024) and torch.equal(back.view(-1).view(torch.int32), want.view(torch.int32))
        tk2.release()
    # a damaged sparse blob is refused on the host, nothing is launched
    tk = a.swap_out(relu, cs.POLICY_SPARSE)
    blob = tk.export()
    tk.release()
    L = cs.sparse_layout(n)
    bad = blob.copy()
    bad[64 + L.tile_off + 4:64 + L.tile_off + 8] = np.frombuffer(np.uint32(n).tobytes(), dtype=np.uint8)
    with pytest.raises(cs.CswapError):
        b.import_blob(bad)
    a.sync()
    b.sync()
    assert a.stats()["pinned_in_use"] == 0 and b.stats()["pinned_in_use"] == 0
    a.close()
    b.close()


def test_zfp_matches_codec(cs, mgr):
    import torch
    t = torch.from_numpy(util.tanh_normal(4 << 20, 2)).cuda()
    want = cs.zfp_decompress(cs.zfp_compress(t, 512), t.numel(), 512)
    tk = mgr.swap_out(t, cs.POLICY_ZFP)
    mgr.sync()
    assert mgr.out_done(tk)
    back = mgr.swap_in(tk)
    torch.cuda.synchronize()
    assert torch.equal(back, want)
    assert tk.info()["moved_bytes"] == t.numel()  # rate 8: one byte per value
    tk.release()


def test_sparse_exact_and_sized(cs, mgr):
    import torch
    a = util.relu_normal(4 << 20, 0.75, 3)
    a[::9] = -0.0
    t = torch.from_numpy(a).cuda()
    tk = mgr.swap_out(t, cs.POLICY_SPARSE)
    back = mgr.swap_in(tk)
    torch.cuda.synchronize()
    assert torch.equal(back.view(torch.int32), t.view(torch.int32))
    info = tk.info()
    nnz = int(torch.count_nonzero(t.view(torch.int32)).item())
    assert info["complete"] and info["moved_bytes"] == cs.sparse_packed_bytes(t.numel(), nnz)
    tk.release()
    assert mgr.stats()["pinned_in_use"] == 0


def test_zfp_odd_sizes(cs, mgr):
    """Less than one 32x32 slab: raw.  Otherwise the whole slabs go through the
    codec and the values past the last slab travel as they are."""
    import torch
    t = torch.from_numpy(util.normal(1000, 4)).cuda()
    tk = mgr.swap_out(t, cs.POLICY_ZFP)
    assert tk.info()["policy"] == cs.POLICY_RAW
    assert torch.equal(mgr.swap_in(tk), t)
    tk.release()
    for n in (1024 + 1, 5 * 1024 + 777, 300 * 1024 + 1023):
        t = torch.tanh(torch.from_numpy(util.normal(n, n)).cuda())
        whole = n // 1024 * 1024
        tk = mgr.swap_out(t, cs.POLICY_ZFP)
        info = tk.info()
        assert info["policy"] == cs.POLICY_ZFP
        assert info["moved_bytes"] == cs.zfp_max_bytes(32, 32, n // 1024, 512) + 4 * (n - whole)
        back = mgr.swap_in(tk)
        torch.cuda.synchronize()
        want = cs.zfp_decompress(cs.zfp_compress(t[:whole].contiguous(), 512), whole, 512)
        assert torch.equal(back[:whole], want) and torch.equal(back[whole:], t[whole:])
        blob = tk.export()
        tk.release()
        tk2 = mgr.import_blob(blob)
        assert torch.equal(mgr.swap_in(tk2), back)
        tk2.release()


def test_many_tensors_interleaved_with_compute(cs, mgr):
    """Swap-outs overlap later compute; swap-ins come back in reverse order with prefetch."""
    import torch
    xs, tks = [], []
    w = torch.randn(512, 512, device="cuda")
    for i in range(12):
        x = torch.relu(torch.randn(1 << 20, device="cuda") - 0.5)
        pol = [cs.POLICY_RAW, cs.POLICY_SPARSE, cs.POLICY_ZFP][i % 3]
        tks.append(mgr.swap_out(x, pol))
        xs.append(x.clone() if pol != cs.POLICY_ZFP else cs.zfp_decompress(cs.zfp_compress(x, 512), x.numel(), 512))
        del x
        w = w @ w.t() * 1e-3  # unrelated compute on the main stream
    for i in reversed(range(12)):
        if i > 0:
            mgr.prefetch(tks[i - 1])
        back = mgr.swap_in(tks[i])
        assert torch.equal(back.view(torch.int32), xs[i].view(torch.int32)), i
        tks[i].release()
    s = mgr.stats()
    assert s["swap_outs"] == 12 and s["swap_ins"] == 12
    assert s["moved_bytes_out"] < s["raw_bytes_out"]
    assert s["pinned_in_use"] == 0 and s["staging_in_use"] == 0


def test_pool_exhaustion_reports_nomem(cs):
    import torch
    m = cs.SwapManager(pinned_bytes=1 << 20, staging_bytes=1 << 20)
    t = torch.zeros(1 << 20, device="cuda")  # 4 MiB > pool
    with pytest.raises(cs.CswapError) as e:
        m.swap_out(t, cs.POLICY_RAW)
    assert e.value.status == 4
    small = torch.ones(1 << 16, device="cuda")
    tk = m.swap_out(small, cs.POLICY_RAW)  # the manager is still usable
    assert torch.equal(m.swap_in(tk), small)
    tk.release()
    m.close()


def test_cost_model_fit_and_decide(cs, mgr, tmp_path):
    cm = cs.CostModel.fit(mgr)
    d = cm.as_dict()
    assert d["d2h_bps"] > 1e9 and d["h2d_bps"] > 1e9
    assert d["zfp_enc_b"] > 0 and d["sparse_enc_b"] > 0
    n = 8 << 20
    link_bound = [
        cs.TensorDesc(n, zero_fraction=0.9, lossy_ok=False, ready_s=1e-4, need_s=1.5e-3),
        cs.TensorDesc(n, zero_fraction=0.0, lossy_ok=True, ready_s=3e-4, need_s=1.0e-3),
        cs.TensorDesc(n, zero_fraction=0.0, lossy_ok=False, ready_s=5e-4, need_s=0.5e-3),
        cs.TensorDesc(1000, zero_fraction=0.0, lossy_ok=True, ready_s=6e-4, need_s=0.1e-3),
    ]
    pol, exp = cm.decide(link_bound, 1e-3)
    assert pol[0] == cs.POLICY_SPARSE       # very sparse, lossless only
    assert pol[1] == cs.POLICY_ZFP          # dense, loss allowed, link saturated
    assert pol[2] == cs.POLICY_RAW          # dense and lossless: nothing helps
    assert pol[3] == cs.POLICY_RAW          # not a multiple of 1024: ZFP not applicable
    hidden = [cs.TensorDesc(1 << 18, 0.9, True, ready_s=1e-3 * i, need_s=1e-2 * (4 - i)) for i in range(4)]
    pol_h, exp_h = cm.decide(hidden, 1e-2)
    # everything hides behind compute either way; the tie goes to the smaller payload (sparse at 90 % zeros)
    assert pol_h == [cs.POLICY_SPARSE] * 4 and sum(exp_h) == 0.0
    path = tmp_path / "policy.json"
    cm.save(str(path), pol)
    cm2, pol2 = cs.CostModel.load(str(path))
    assert pol2 == pol and cm2.as_dict() == d
    path.write_text("{ truncated")
    with pytest.raises(Exception):
        cs.CostModel.load(str(path))


def _small_net(torch):
    torch.manual_seed(0)
    import torch.nn as nn
    layers = [nn.Conv2d(3, 32, 3, padding=1), nn.ReLU(), nn.Conv2d(32, 32, 3, padding=1), nn.ReLU(),
              nn.MaxPool2d(2), nn.Conv2d(32, 64, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(64 * 16 * 16, 10)]
    return nn.Sequential(*layers).cuda()


def _step(cs, torch, net, x, y, policy_for, planner=1, give_producers=False):
    """One forward/backward with every layer wrapped in pre/post; returns loss and grads."""
    exe = cs.Execution()
    n = len(net)
    exe.init_(n + 1)
    exe.policy_ = planner
    for i in range(n):
        exe.begin_stage[i] = i + 1
        exe.policy[i] = policy_for(i, net[i])
    for p in net.parameters():
        p.grad = None
    exe.preforward()
    h = x
    for i, layer in enumerate(net):
        lt = cs.LayerType.CONV if isinstance(layer, torch.nn.Conv2d) else cs.LayerType.ACT
        exe.pre(h, lt)
        out = layer(h)
        exe.post(h, out, lt, False, layer if give_producers else None)
        h = out
    exe.postforward()
    loss = torch.nn.functional.cross_entropy(h, y)
    loss.backward()
    torch.cuda.synchronize()
    grads = [p.grad.clone() for p in net.parameters()]
    stats = exe.mgr.stats()
    exe.mgr.close()
    return float(loss.detach()), grads, stats, exe


def test_execution_lossless_policies_do_not_change_training(cs):
    import torch
    net = _small_net(torch)
    x = torch.randn(64, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda")
    torch.backends.cudnn.deterministic = True
    base_loss, base_grads, _, _ = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_KEEP)
    for pol in (cs.POLICY_RAW, cs.POLICY_SPARSE):
        loss, grads, stats, exe = _step(cs, torch, net, x, y, lambda i, l: pol)
        # conv outputs feed ReLUs, which keep their own output: nobody saves them, so they are not copied out
        assert exe.swapped_tensors >= 5 and exe.skipped_unsaved >= 3
        # everything that went out was needed again: swapped in, or taken back before its copy had run
        assert stats["swap_ins"] + exe.mgr.reclaimed_tensors == exe.swapped_tensors
        assert loss == base_loss
        for g, b in zip(grads, base_grads):
            assert torch.equal(g, b)
    # sparse moves fewer bytes than raw on the ReLU outputs
    _, _, s_raw, _ = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_RAW if isinstance(l, torch.nn.ReLU) else 0)
    _, _, s_sp, _ = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_SPARSE if isinstance(l, torch.nn.ReLU) else 0)
    assert s_sp["moved_bytes_out"] < 0.8 * s_raw["moved_bytes_out"]


def test_execution_drop_and_recompute(cs):
    """Policy 1 (Execution.h:243-247): the tensor is let go without a copy and
    rebuilt in backward from its producer; training is unchanged bit for bit.
    Chains of dropped tensors rebuild each other; without a producer the
    tensor stays."""
    import torch
    net = _small_net(torch)
    x = torch.randn(64, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda")
    torch.backends.cudnn.deterministic = True
    base_loss, base_grads, _, _ = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_KEEP)
    # every wrapped tensor dropped: each rebuild pulls in the one before it
    loss, grads, stats, exe = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_DROP, give_producers=True)
    assert exe.dropped_tensors >= 6 and exe.recomputed_tensors >= 4 and stats["swap_outs"] == 0
    assert loss == base_loss
    for g, b in zip(grads, base_grads):
        assert torch.equal(g, b)
    # mixed: ReLU outputs dropped, the rest swapped raw, so rebuilding a ReLU output swaps its input in
    loss, grads, stats, exe = _step(cs, torch, net, x, y,
                                    lambda i, l: cs.POLICY_DROP if isinstance(l, torch.nn.ReLU) else cs.POLICY_RAW,
                                    give_producers=True)
    assert exe.dropped_tensors >= 3 and exe.recomputed_tensors >= 2 and stats["swap_ins"] >= 2
    assert loss == base_loss
    for g, b in zip(grads, base_grads):
        assert torch.equal(g, b)
    # no producer given: policy 1 leaves the tensors where they are
    loss, grads, stats, exe = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_DROP)
    assert exe.dropped_tensors == 0 and exe.recomputed_tensors == 0 and loss == base_loss


def test_execution_baseline_planners(cs):
    """policy_ 3 (vDNN) swaps exactly the inputs of conv layers raw; policy_ 4
    (SuperNeurons) also drops and rebuilds the inputs of the other layers
    (Execution.h:70,243,248).  Both leave training unchanged."""
    import torch
    net = _small_net(torch)
    n_conv = sum(isinstance(l, torch.nn.Conv2d) for l in net)
    x = torch.randn(64, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda")
    torch.backends.cudnn.deterministic = True
    base_loss, base_grads, _, _ = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_KEEP)
    loss, grads, stats, exe = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_KEEP, planner=3, give_producers=True)
    # the first conv reads the network input, which no layer produced: nothing to swap there
    assert stats["swap_outs"] == n_conv - 1 and exe.dropped_tensors == 0
    assert loss == base_loss and all(torch.equal(g, b) for g, b in zip(grads, base_grads))
    loss, grads, stats, exe = _step(cs, torch, net, x, y, lambda i, l: cs.POLICY_KEEP, planner=4, give_producers=True)
    assert stats["swap_outs"] == n_conv - 1 and exe.dropped_tensors >= 2 and exe.recomputed_tensors >= 1
    assert loss == base_loss and all(torch.equal(g, b) for g, b in zip(grads, base_grads))


def test_reference_python_hook_names(cs):
    """The torch.cswap* call pattern of the reference's model zoo
    (CIFAR10/models/vgg.py:23-46) on stock PyTorch."""
    import types
    import torch
    import cswap_b200.compat as compat
    ns = types.SimpleNamespace()
    compat.install(ns)
    net = _small_net(torch)
    x = torch.randn(64, 3, 32, 32, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda")
    torch.backends.cudnn.deterministic = True

    def run(type_for):
        for p in net.parameters():
            p.grad = None
        ns.cswapinit()
        out = x
        for layer in net:
            t = type_for(layer)
            pre = out
            ns.cswappre(pre, t)
            out = layer(pre)
            ns.cswappost(pre, out, t)
        loss = torch.nn.functional.cross_entropy(out, y)
        loss.backward()
        torch.cuda.synchronize()
        return float(loss.detach()), [p.grad.clone() for p in net.parameters()]

    ns.cswapinit_()
    ns.cswapsetratio(512)
    base = run(lambda l: 0)
    mgr = compat.execution().mgr
    before = mgr.stats()["swap_outs"]
    got = run(lambda l: 2 if isinstance(l, torch.nn.Conv2d) else 3)   # "2 = vDNN" on conv inputs, ZVC elsewhere
    assert mgr.stats()["swap_outs"] - before >= 4
    assert got[0] == base[0] and all(torch.equal(a, b) for a, b in zip(got[1], base[1]))
    lossy = run(lambda l: 6 if isinstance(l, torch.nn.Conv2d) else 0)  # "6 = ZFP"
    assert abs(lossy[0] - base[0]) < 1e-3 and not all(torch.equal(a, b) for a, b in zip(lossy[1], base[1]))
    compat.execution().postforward()
    mgr.close()


def test_execution_zfp_equals_codec_applied_to_activations(cs):
    """With policy 6 on one tensor, backward sees exactly decode(encode(x))."""
    import torch
    torch.manual_seed(1)
    lin = torch.nn.Linear(1024, 1024).cuda()
    x0 = torch.randn(256, 1024, device="cuda", requires_grad=True)
    h = torch.tanh(x0)  # id 0
    exe = cs.Execution()
    exe.init_(4)
    exe.policy[0] = cs.POLICY_ZFP
    exe.begin_stage[0] = 1
    exe.preforward()
    exe.pre(x0)
    h = torch.tanh(x0)
    exe.post(x0, h)          # h.tensor_id = 0
    exe.pre(h)               # index 1 == begin_stage[0] -> swap h out with ZFP
    out = lin(h)
    exe.post(h, out)
    exe.postforward()
    h_ref = h.detach().clone()
    del h
    out.sum().backward()
    torch.cuda.synchronize()
    lossy = cs.zfp_decompress(cs.zfp_compress(h_ref.view(-1), 512), h_ref.numel(), 512).view_as(h_ref)
    # dL/dW = ones^T @ h : computed from the decompressed activation
    want = torch.ones(256, 1024, device="cuda").t() @ lossy
    assert torch.allclose(lin.weight.grad, want, rtol=1e-5, atol=1e-4)
    assert not torch.allclose(lossy, h_ref)  # the activation really went through the lossy codec
    # tanh's own backward used the same record (1 - h^2 with the lossy h)
    want_x = (torch.ones(256, 1024, device="cuda") @ lin.weight.detach()) * (1 - lossy * lossy)
    assert torch.allclose(x0.grad, want_x, rtol=1e-4, atol=1e-5)
    assert exe.mgr.stats()["swap_ins"] == 1
    exe.mgr.close()


def test_profile_and_make_policy(cs):
    import torch
    net = _small_net(torch)
    x = torch.randn(128, 3, 32, 32, device="cuda")
    exe = cs.Execution(mgr=cs.SwapManager(pinned_bytes=512 << 20, staging_bytes=128 << 20))
    exe.init_(len(net) + 1)
    exe.profile = True
    exe.preforward()
    h = x.requires_grad_()
    for i, layer in enumerate(net):
        lt = cs.LayerType.CONV if isinstance(layer, torch.nn.Conv2d) else cs.LayerType.ACT
        exe.pre(h, lt)
        out = layer(h)
        exe.post(h, out, lt, False, layer)
        h = out
    exe.postforward()
    prof = exe.finish_profile()
    assert len(prof) == len(net) and all(p["time_s"] >= 0 for p in prof.values())
    assert not prof[0]["saved"] and prof[1]["saved"]  # conv output feeds a ReLU; the ReLU output is kept
    assert 0.3 < prof[1]["zero_fraction"] < 0.7  # first ReLU output
    cm = cs.CostModel.fit(exe.mgr)
    pol = exe.make_policy(prof, cm, min_bytes=1 << 16)
    assert len(pol) >= len(net)
    assert set(pol) <= {0, 2, 3, 6}
    assert exe.begin_stage[1] == 2  # ReLU output is consumed by the next conv
    assert pol[0] == 0               # nothing keeps the first conv's output: not a candidate
    # the model's table and its ZFP-eager neighbour; the run-off installs whichever "runs" faster
    cands = exe.policy_candidates(prof, cm, lossy_ids=[1, 3, 4, 6], min_bytes=1 << 16)
    assert set(cands) == {"model", "zfp_where_allowed"} and cands["model"][1] in (2, 3, 6)
    assert all(cands["zfp_where_allowed"][i] == 6 for i in (1, 3, 4, 6))
    fake = iter([0.0, 3.0, 0.0, 2.0])       # seconds returned for (settle, timed) x (model, neighbour)
    assert exe.refine_policy(cands, lambda k: next(fake)) == "zfp_where_allowed"
    assert exe.policy[:len(net)] == cands["zfp_where_allowed"][:len(net)]
    fake = iter([0.0, 1.0, 0.0, 2.0])
    assert exe.refine_policy(cands, lambda k: next(fake)) == "model"
    assert exe.policy[:len(net)] == cands["model"][:len(net)]
    # swap-or-recompute table in the manner of Capuchin: raw swaps and rebuilds only, planner code 2
    cap = exe.make_policy_capuchin(prof, cm, min_bytes=1 << 16)
    assert set(cap) <= {0, 1, 2} and exe.policy_ == 2 and cap[1] in (1, 2) and cap[0] == 0
    # a link a thousand times slower makes every copy stall: everything that can be rebuilt is
    slow = cs.CostModel.fit(exe.mgr)
    slow.c.d2h_bps /= 1000.0
    slow.c.h2d_bps /= 1000.0
    cap_slow = exe.make_policy_capuchin(prof, slow, min_bytes=1 << 16)
    assert cap_slow.count(1) > cap.count(1) and cap_slow.count(1) >= 2
    exe.mgr.close()


def test_staged_payload_kept_until_the_pool_needs_room(cs):
    """A compressed payload stays in device staging after its copy out: a
    swap-in that finds it there moves nothing over the link; with the pool too
    small for all of them the oldest make room (and come back over the link);
    csw_mgr_keep_staged(0) or csw_mgr_sync drop the kept copies.  The tensors
    that come back are the same bits in every case."""
    import time
    import torch

    def settle(m, tickets):
        # wait (without csw_mgr_sync, which drops the kept copies) until the copies out are done
        torch.cuda.synchronize()
        for _ in range(2000):
            if all(m.out_done(tk) for tk in tickets):
                break
            time.sleep(0.001)
        time.sleep(0.05)  # the copies out (4 MiB each) trail the codec; no call waits for them without dropping the kept copies
        m.stats()         # a call that runs the manager's housekeeping

    ts = [torch.from_numpy(util.tanh_normal(4 << 20, seed=i)).cuda() for i in range(4)]  # 16 MiB each, 4 MiB coded
    want = []
    ref = cs.SwapManager(pinned_bytes=256 << 20, staging_bytes=64 << 20)
    ref.keep_staged(False)
    for t in ts:
        tk = ref.swap_out(t, cs.POLICY_ZFP)
        settle(ref, [tk])
        want.append(ref.swap_in(tk).clone())
        tk.release()
    torch.cuda.synchronize()
    s = ref.stats()
    assert s["moved_bytes_in"] == s["moved_bytes_out"] == 4 * (4 << 20)  # released at once: all of it crossed again
    ref.close()

    m = cs.SwapManager(pinned_bytes=256 << 20, staging_bytes=64 << 20)
    tks = [m.swap_out(t, cs.POLICY_ZFP) for t in ts]
    settle(m, tks)
    for tk, w in zip(reversed(tks), reversed(want)):
        assert torch.equal(m.swap_in(tk), w)
    torch.cuda.synchronize()
    assert m.stats()["moved_bytes_in"] == 0           # all four were still staged
    for tk in tks:
        tk.release()
    m.close()

    small = cs.SwapManager(pinned_bytes=256 << 20, staging_bytes=10 << 20)  # room for two payloads
    tks = []
    for t in ts:
        tks.append(small.swap_out(t, cs.POLICY_ZFP))
        settle(small, tks)
    for tk, w in zip(reversed(tks), reversed(want)):
        assert torch.equal(small.swap_in(tk), w)
    torch.cuda.synchronize()
    got = small.stats()["moved_bytes_in"]
    assert 0 < got < 4 * (4 << 20)                    # the newest were kept, the oldest had to make room
    for tk in tks:
        tk.release()
    small.close()

    m = cs.SwapManager(pinned_bytes=256 << 20, staging_bytes=64 << 20)
    tk = m.swap_out(ts[0], cs.POLICY_ZFP)
    m.sync()                                          # everything on the host only
    assert m.stats()["staging_in_use"] == 0
    assert torch.equal(m.swap_in(tk), want[0])
    torch.cuda.synchronize()
    assert m.stats()["moved_bytes_in"] == 4 << 20
    tk.release()
    m.close()


def test_raw_copies_wait_in_the_managers_queue(cs):
    """Raw copies out are handed to the copy stream two at a time; a ticket
    given up while its copy still waits is never copied (csw_swap_out_cancel),
    and one that is not given up comes back bit for bit."""
    import torch
    m = cs.SwapManager(pinned_bytes=512 << 20, staging_bytes=16 << 20)
    ts = [torch.randn(1 << 20, device="cuda") for _ in range(8)]    # 4 MiB each
    torch.cuda.synchronize()
    torch.cuda._sleep(int(4e8))          # the GPU is busy: no copy can start yet (it waits for this stream)
    tks = [m.swap_out(t, cs.POLICY_RAW) for t in ts]
    assert not any(m.out_done(tk) for tk in tks)
    cancelled = sum(m._cancel(tk) for tk in reversed(tks))
    assert cancelled == 6                # two had been handed to the copy stream already
    assert [tk.alive for tk in tks] == [True, True] + [False] * 6
    back = m.swap_in(tks[0])
    torch.cuda.synchronize()
    assert torch.equal(back, ts[0])
    for tk in tks[:2]:
        tk.release()
    m.sync()
    s = m.stats()
    assert s["moved_bytes_out"] == 2 * (4 << 20) and s["pinned_in_use"] == 0
    m.close()

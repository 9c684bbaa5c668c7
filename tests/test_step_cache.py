"""Block-level step cache: the host-side state machine against vectors recorded from the reference's DBCache (CPU),
and the CUDA residual statistics against the eager expressions (GPU)."""

import pytest
import torch

from ksanadit_b200.step_cache import B200DBCache, DBCacheConfig, relative_l1


def _eager_diff(x_new, x_old, prev):
    """The reference's own expressions (dbcache.py:228-239,301-306), used as the statistics provider of the state machine."""
    r = x_new - x_old
    if prev is None or prev.shape != r.shape:
        return r, None
    cm, pm = torch.abs(r).mean() + 1e-8, torch.abs(prev).mean() + 1e-8
    return r, float(torch.abs(r - prev).mean() / ((cm + pm) / 2))


def _toy(golden, device="cpu"):
    g = golden["dbcache"]
    ws = [w.to(device) for w in g["weights"]]
    blocks = [(lambda x, scale=1.0, w=w: x + torch.tanh(x.float() @ w).to(x.dtype) * scale) for w in ws]
    return g, blocks, g["x"].to(device)


def _run(cache, blocks, x):
    outs = []
    for step in range(14):
        for phase in ("cond", "uncond"):
            xin = (x * (1 + 0.02 * step) + (0.3 if phase == "uncond" else 0)).to(torch.bfloat16)
            outs.append(cache(phase, xin.clone(), step, 1000 - step * 10, blocks, scale=1.0 + 0.001 * step))
    return torch.stack(outs)


def test_state_machine_reproduces_reference_dbcache(golden):
    g, blocks, x = _toy(golden)
    for case in g["cases"]:
        cache = B200DBCache(DBCacheConfig(**case["cfg"]), diff_fn=_eager_diff)
        outs = _run(cache, blocks, x)
        assert torch.equal(outs, case["outs"]), case["cfg"]
        s = cache.get_stats_summary()
        assert (s["cond_cached_steps"], s["uncond_cached_steps"]) == (case["cond_cached"], case["uncond_cached"])
        assert torch.allclose(torch.tensor(cache.diff_history), case["diffs"], rtol=0, atol=0)
        cache.reset()
        assert cache.step == 0 and cache.state["cond"].first_residual is None


def test_limits_and_validation():
    with pytest.raises(ValueError):
        B200DBCache(DBCacheConfig(fn_compute_blocks=4, bn_compute_blocks=4, num_blocks=6))
    c = B200DBCache(DBCacheConfig(max_warmup_steps=3, warmup_interval=2, num_blocks=2), diff_fn=_eager_diff)
    assert c._is_warmup() and c.valid_for("cond") is False  # warm-up and nothing cached yet
    c.step = 1
    assert not c._is_warmup()  # warm-up steps are every second step below max_warmup_steps
    assert c(phase="cond", x=torch.ones(2, 8), step_iter=0, timestep=5, blocks=None).sum() == 16
    with pytest.raises(Exception):  # the default statistics provider has no CPU path
        B200DBCache(DBCacheConfig(num_blocks=1, max_warmup_steps=0))("cond", torch.ones(2, 8, dtype=torch.bfloat16), 0, 1, [lambda x: x + 1])
    sums = torch.tensor([3.0, 8.0, 8.0])
    assert relative_l1(sums, 8, torch.float32) == pytest.approx(0.375)


@pytest.mark.gpu
def test_device_statistics_match_eager_and_drive_same_decisions(golden):
    from ksanadit_b200 import _lib, ops
    g = torch.Generator().manual_seed(3)
    a = torch.randn(333, 256, generator=g).to(torch.bfloat16).cuda()
    b = (a.float() + 0.1 * torch.randn(333, 256, generator=g).cuda()).to(torch.bfloat16)
    prev = (0.1 * torch.randn(333, 256, generator=g)).to(torch.bfloat16).cuda()
    res, sums = ops.residual_diff(b, a, prev)
    r = b - a
    assert torch.equal(res, r)
    want = torch.stack([torch.abs(r - prev).float().sum(), r.abs().float().sum(), prev.abs().float().sum()])
    assert torch.allclose(sums, want, rtol=1e-5)
    eager = float(torch.abs(r - prev).mean() / (((r.abs().mean() + 1e-8) + (prev.abs().mean() + 1e-8)) / 2))
    assert relative_l1(sums, r.numel(), torch.bfloat16) == pytest.approx(eager, rel=1e-2)
    res2, sums2 = ops.residual_diff(b, a, None, want_residual=False)
    assert res2 is None and float(sums2[0]) == 0.0 and float(sums2[2]) == 0.0 and torch.allclose(sums2[1], want[1], rtol=1e-5)
    # the whole cache on the GPU with the kernel's statistics: same hits and same outputs as with the eager expressions
    gold, blocks, x = _toy(golden, "cuda")
    for case in gold["cases"]:
        dev_cache = B200DBCache(DBCacheConfig(**case["cfg"]))
        outs = _run(dev_cache, blocks, x)
        s = dev_cache.get_stats_summary()
        assert (s["cond_cached_steps"], s["uncond_cached_steps"]) == (case["cond_cached"], case["uncond_cached"])
        # the toy blocks themselves (tanh, fp32 matmul) differ in the last bits between the CPU and the GPU, and bf16
        # rounding carries that through six blocks: the recorded outputs are matched to a few bf16 steps
        assert torch.allclose(outs.cpu().float(), case["outs"].float(), atol=8e-2, rtol=3e-2)
    _lib.assert_device_ok()


@pytest.mark.gpu
def test_denoise_step_through_the_cache_skips_blocks_and_stays_close():
    """A 4-block Wan-shaped stack over slowly drifting inputs: after the warm-up the cache replaces the last three
    blocks by their remembered residual, with fewer launches and a result close to the full computation."""
    from ksanadit_b200 import _lib, ops
    from ksanadit_b200.wan_block import B200WanDenoiseStep
    dim, ffn, heads, grid = 256, 768, 2, (1, 8, 8)
    cache = B200DBCache(DBCacheConfig(fn_compute_blocks=1, bn_compute_blocks=0, residual_diff_threshold=0.5, max_warmup_steps=2,
                                      max_cached_steps=8, max_continuous_cached_steps=2, num_blocks=4))
    cached = B200WanDenoiseStep(4, dim, ffn, heads, seed=5, step_cache=cache)
    plain = B200WanDenoiseStep(4, dim, ffn, heads, seed=5)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 64, dim, generator=g).to(torch.bfloat16).cuda()
    e = (torch.randn(1, 1, 6, dim, generator=g) * 0.1).to(torch.bfloat16).cuda()
    c = torch.randn(1, 16, dim, generator=g).to(torch.bfloat16).cuda()
    hits = 0
    with torch.no_grad():
        for step in range(6):
            xin = (x.float() * (1 + 0.002 * step)).to(torch.bfloat16)
            n0 = ops.STATS.kernels
            y = cached(xin, e, [grid], c, phase="cond", step_iter=step, timestep=1000 - step)
            n_cached = ops.STATS.kernels - n0
            ref = plain(xin, e, [grid], c)
            n_plain = ops.STATS.kernels - n0 - n_cached
            if n_cached < n_plain:
                hits += 1
                a, b = y.float().flatten().double(), ref.float().flatten().double()
                assert float((a @ b) / (a.norm() * b.norm())) > 0.999
            else:
                assert torch.equal(y, ref)
    _lib.assert_device_ok()
    assert hits == cache.get_stats_summary()["cond_cached_steps"] and hits >= 2

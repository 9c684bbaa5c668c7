"""A step captured into one CUDA graph must reproduce the eagerly launched step bit for bit, also on new inputs."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wan_blocks_graph_replay_equals_eager():
    from ksanadit_b200 import _lib
    from ksanadit_b200.graph import StepGraph
    from ksanadit_b200.wan_block import B200WanDenoiseStep
    dim, ffn, heads, grid = 512, 1024, 4, (2, 8, 10)
    L = grid[0] * grid[1] * grid[2]
    model = B200WanDenoiseStep(2, dim, ffn, heads, device="cuda", seed=3)
    g = torch.Generator().manual_seed(1)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    x, e, c = mk(1, L, dim), mk(1, 1, 6, dim) * 0.1, mk(1, 24, dim)
    fn = lambda x_, e_, c_: model(x_, e_, [grid], c_)
    graph = StepGraph(fn, (x, e, c))
    assert graph.kernels_per_replay > 0
    for seed in (2, 3):
        g = torch.Generator().manual_seed(seed)
        x2, e2, c2 = mk(1, L, dim), mk(1, 1, 6, dim) * 0.1, mk(1, 24, dim)
        with torch.no_grad():
            ref = fn(x2.clone(), e2, c2).clone()
        got = graph(x2, e2, c2).clone()
        _lib.assert_device_ok()
        assert torch.equal(ref, got)


def test_qwen_block_graph_replay_equals_eager():
    from ksanadit_b200 import _lib
    from ksanadit_b200.graph import StepGraph
    from ksanadit_b200.qwen_block import B200QwenBlock
    dim, heads, ffn, grid, Lt = 512, 4, 1024, (1, 8, 12), 40
    blk = B200QwenBlock(dim, heads, ffn).random_init(9)
    g = torch.Generator().manual_seed(4)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    img, txt, temb = mk(1, grid[1] * grid[2], dim), mk(1, Lt, dim), mk(1, dim)

    def fn(i, t, e):
        t2, i2 = blk(i, t, e, img_grid=grid)
        return torch.cat([t2, i2], dim=1)

    graph = StepGraph(fn, (img, txt, temb))
    img2, txt2, temb2 = mk(1, grid[1] * grid[2], dim), mk(1, Lt, dim), mk(1, dim)
    with torch.no_grad():
        ref = fn(img2.clone(), txt2.clone(), temb2).clone()
    got = graph(img2, txt2, temb2).clone()
    _lib.assert_device_ok()
    assert torch.equal(ref, got)


@pytest.mark.parametrize("text_stream", [False, True])
def test_qwen_step_driver_equals_the_block_loop(text_stream):
    """B200QwenDenoiseStep launches every block's modulation GEMM ahead on a stream of its own and (optionally) the text
    stream's kernels beside the image stream's: same bits as calling the blocks one after the other, eagerly and as one
    CUDA graph on new inputs."""
    from ksanadit_b200 import _lib
    from ksanadit_b200.graph import StepGraph
    from ksanadit_b200.qwen_block import B200QwenBlock, B200QwenDenoiseStep
    dim, heads, ffn, grid, Lt = 512, 4, 1024, (1, 8, 12), 40
    Li = grid[1] * grid[2]
    blocks = [B200QwenBlock(dim, heads, ffn).random_init(20 + i) for i in range(3)]
    drv = B200QwenDenoiseStep(blocks, text_stream=text_stream)
    g = torch.Generator().manual_seed(6)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()

    def loop(i, t, e):
        for b in blocks:
            t, i = b(i, t, e, img_grid=grid)
        return torch.cat([t, i], dim=1)

    def driven(i, t, e):
        t2, i2 = drv(i, t, e, img_grid=grid)
        return torch.cat([t2, i2], dim=1)

    img, txt, temb = mk(1, Li, dim), mk(1, Lt, dim), mk(1, dim)
    with torch.no_grad():
        ref = loop(img, txt, temb)
        got = driven(img, txt, temb)
    torch.cuda.synchronize()
    _lib.assert_device_ok()
    assert torch.equal(ref, got)
    graph = StepGraph(driven, (img, txt, temb))
    img2, txt2, temb2 = mk(1, Li, dim), mk(1, Lt, dim), mk(1, dim)
    with torch.no_grad():
        ref2 = loop(img2, txt2, temb2).clone()
    got2 = graph(img2, txt2, temb2).clone()
    _lib.assert_device_ok()
    assert torch.equal(ref2, got2)


def test_step_graph_rejects_other_shapes():
    from ksanadit_b200 import _lib
    from ksanadit_b200.graph import StepGraph
    from ksanadit_b200 import ops
    x = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    graph = StepGraph(lambda t: ops.quant_fp8_rowwise(t)[0], (x,))
    with pytest.raises(_lib.KsanaB200Error):
        graph(x[:32])


def test_torch_library_ops_match_the_direct_calls():
    import ksanadit_b200.torch_ops  # noqa: F401
    from ksanadit_b200 import ops
    from ksanadit_b200.linear import B200Fp8Linear, quantize_weight_per_channel
    g = torch.Generator().manual_seed(8)
    x = torch.randn(3, 50, 256, generator=g).to(torch.bfloat16).cuda()
    lin = B200Fp8Linear(256, 128, device="cuda", dtype=torch.bfloat16)
    wq, s = quantize_weight_per_channel((torch.randn(128, 256, generator=g) * 0.02).cuda())
    lin.weight = torch.nn.Parameter(wq, requires_grad=False)
    lin.scale_weight = torch.nn.Parameter(s, requires_grad=False)
    lin.bias = torch.nn.Parameter((torch.randn(128, generator=g) * 0.1).to(torch.bfloat16).cuda(), requires_grad=False)
    assert torch.equal(torch.ops.ksana_b200.fp8_linear(x, lin.weight, lin.scale_weight, lin.bias), lin(x))
    q, k, v = (torch.randn(200, 2, 128, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    assert torch.equal(torch.ops.ksana_b200.sage_attention(q, k, v), ops.sage_attention(q, k, v))

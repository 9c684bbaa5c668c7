"""CPU tests: the host-side mirrors of KsanaDiT's operator contracts and the C-ABI surface (no GPU work)."""

import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from ksanadit_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "ksana_b200.h")).read()
    declared = set(re.findall(r"\b(ksb_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))
    assert _lib.load().ksb_version() >= 100


def test_no_cpu_fallback_and_argument_checks():
    from ksanadit_b200 import _lib, ops
    with pytest.raises(_lib.KsanaB200Error):
        ops.quant_fp8_rowwise(torch.zeros(4, 32, dtype=torch.bfloat16))
    with pytest.raises(_lib.KsanaB200Error):
        ops.sage_attention(*(torch.zeros(8, 1, 128, dtype=torch.bfloat16) for _ in range(3)))
    lib = _lib.load()
    # rejected before any CUDA call: null pointers / bad shapes return -1 and set a message
    assert lib.ksb_quant_fp8_rowwise(None, 0, 4, 24, 24, None, None, None) == -1
    assert b"multiple of 16" in lib.ksb_last_error()
    assert lib.ksb_fp8_gemm(None, None, None, None, None, 4, 8, 16, None, 0, 8, 0, None, 0, None, 0, None) == -1
    assert lib.ksb_sage_attn(None, None, None, None, None, None, 1, 1, 1, None, None, None, None, 0, 128, 128, None, 0, 0, None) == -1
    assert lib.ksb_sage_kmean_scratch_floats(75600, 40, 128) == 148 * 40 * 128


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "ksanadit_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("# oracle", ""), f"{f} mentions the oracle"


def test_linear_contract_and_state_dict_loading():
    from ksanadit_b200 import linear
    m = linear.B200Fp8Linear(64, 48, bias=True, dtype=torch.bfloat16)
    assert m.weight.dtype == torch.float8_e4m3fn and m.weight.shape == (48, 64) and m.scale_input is None
    w = torch.randn(48, 64) * 0.02
    wq, s = linear.quantize_weight_per_channel(w)
    sd = {"weight": wq, "bias": torch.zeros(48, dtype=torch.bfloat16), "scale_weight": s}
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not missing and not unexpected and m.scale_weight.shape == (48,)
    assert torch.equal(m.weight_scale_vector(), s)
    # per-tensor checkpoints (the reference's granularity) broadcast
    m2 = linear.b200_fp8_ops(scale_input=True)(64, 48)
    assert m2.scale_input is not None and m2.scale_weight.dim() == 0
    m2.load_state_dict({"weight": wq, "bias": torch.zeros(48, dtype=torch.bfloat16), "scale_weight": torch.tensor(0.5),
                        "scale_input": torch.tensor(0.25)}, strict=False)
    assert bool((m2.weight_scale_vector() == 0.5).all())
    with pytest.raises(Exception):
        m(torch.zeros(2, 3, 4, 64, dtype=torch.bfloat16))  # rank 4 is an error, not a silent fallback
    from oracle import quantizers as Qz
    wq_o, s_o = Qz.weight_quant_fp8_channelwise(w)
    assert torch.equal(wq.view(torch.uint8), wq_o.view(torch.uint8)) and torch.equal(s, s_o)


def test_pick_linear_rules():
    from ksanadit_b200 import _lib, linear
    from ksanadit_b200.config import KsanaLinearBackend as LB
    fp8_sd = {"a.weight": torch.zeros(2, 2).to(torch.float8_e4m3fn), "scaled_fp8": torch.zeros(1)}
    cls = linear.pick_linear(torch.bfloat16, fp8_sd, LB.DEFAULT)
    assert issubclass(cls, linear.B200Fp8Linear) and "scaled_fp8" not in fp8_sd
    scaled = {"a.weight": torch.zeros(2, 2).to(torch.float8_e4m3fn), "a.scale_weight": torch.ones(())}
    assert issubclass(linear.pick_linear(torch.bfloat16, scaled, "fp8_gemm"), linear.B200Fp8Linear)
    with pytest.raises(ValueError):
        linear.pick_linear(torch.bfloat16, {"a.weight": torch.zeros(2, 2)}, LB.FP8_GEMM)
    with pytest.raises(_lib.KsanaB200Error):
        linear.pick_linear(torch.bfloat16, {"a.weight": torch.zeros(2, 2)}, LB.DEFAULT)
    assert linear.pick_linear(torch.bfloat16, {"a.weight": torch.zeros(2, 2)}, LB.FP8_GEMM_DYNAMIC) is linear.B200Fp8Linear


def test_qkv_remap_builds_per_channel_scales():
    from ksanadit_b200 import fuse_qkv
    sd = {}
    for i, n in enumerate("qkv"):
        sd[f"blocks.0.self_attn.{n}.weight"] = torch.full((4, 8), float(i + 1)).to(torch.float8_e4m3fn)
        sd[f"blocks.0.self_attn.{n}.bias"] = torch.full((4,), float(i))
        sd[f"blocks.0.self_attn.{n}.scale_weight"] = torch.tensor(0.1 * (i + 1))
    sd["blocks.0.self_attn.o.weight"] = torch.zeros(4, 4)
    out = fuse_qkv.remap_qkv_weights(sd, fuse_qkv.MODEL_QKV_PATTERNS["wan"])
    assert out["blocks.0.self_attn.qkv.weight"].shape == (12, 8)
    assert torch.allclose(out["blocks.0.self_attn.qkv.scale_weight"], torch.tensor([0.1] * 4 + [0.2] * 4 + [0.3] * 4))
    assert out["blocks.0.self_attn.qkv.bias"].tolist() == [0.0] * 4 + [1.0] * 4 + [2.0] * 4
    assert "blocks.0.self_attn.q.weight" not in out and "blocks.0.self_attn.o.weight" in out


def test_attention_backend_contract():
    from ksanadit_b200 import attention
    from ksanadit_b200.config import KsanaAttentionBackend, KsanaAttentionConfig, KsanaRadialSageAttentionConfig
    assert attention.B200SageAttentionImpl.type() == KsanaAttentionBackend.SAGE_ATTN
    assert attention.B200SageAttentionImpl.supports(head_size=64, dtype=torch.bfloat16) is False
    with pytest.raises(ValueError):
        KsanaRadialSageAttentionConfig(decay_factor=1.5)
    with pytest.raises(ValueError):
        KsanaRadialSageAttentionConfig(block_size=32)
    op = attention.pick_attn_op(KsanaAttentionConfig(backend=KsanaAttentionBackend.SAGE_ATTN))(num_heads=2, head_size=128)
    with pytest.raises(ValueError):
        op(torch.zeros(2, 3, 128), torch.zeros(2, 3, 128), torch.zeros(2, 3, 128))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):  # no silent substitution of another backend
            op(*(torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16) for _ in range(3)))


def test_product_radial_mask_matches_reference_vectors(golden):
    from ksanadit_b200 import radial_mask as P
    from oracle import radial_mask as R
    for key, packed in golden["radial_masks"].items():
        vt, nf, bs, decay, s = key.split("_")
        m = P.build_radial_tile_mask(int(s), int(vt), int(nf), int(bs), float(decay))
        ref = np.unpackbits(packed.numpy())[: m.size].reshape(m.shape).astype(bool)
        assert np.array_equal(m, ref), key
    m = R.expand_to_q128_k64(R.bernoulli_frame_mask(5000, 900, 1), 128)
    assert all(np.array_equal(a, b) for a, b in zip(P.compact_tile_lists(m), R.tile_lists(m)))
    assert np.array_equal(P.bernoulli_frame_tile_mask(5000, 900, 1), R.bernoulli_frame_mask(5000, 900, 1))


_A2A_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from ksanadit_b200 import distribute
from oracle import ulysses
dist.init_process_group("gloo", init_method="env://")
r, P = dist.get_rank(), dist.get_world_size()
g = torch.Generator().manual_seed(0)
full = [torch.randn(1, 6, 4, 8, generator=g) for _ in range(P)]       # every rank's [B, L_loc, H, D]
exp_fwd = ulysses.all_to_all_emulated(full, scatter_dim=2, gather_dim=1)
got = distribute.all_to_all(full[r].clone(), scatter_dim=2, gather_dim=1)
assert torch.equal(got, exp_fwd[r]), "all_to_all forward layout"
back = distribute.all_to_all(got, scatter_dim=1, gather_dim=2)
assert torch.equal(back, full[r]), "all_to_all inverse"
# fused three-tensor exchange used by the block path
qkv = [torch.randn(6, 3, 4, 8, generator=g) for _ in range(P)]
h2s = distribute.heads_to_sequence(qkv[r].clone())
exp = torch.cat([t[:, :, r * (4 // P):(r + 1) * (4 // P)] for t in qkv], dim=0)
assert torch.equal(h2s, exp), "heads_to_sequence"
s2h = distribute.sequence_to_heads(h2s[:, 0].contiguous())
assert torch.equal(s2h, qkv[r][:, 0]), "sequence_to_heads"
assert torch.equal(distribute.gather_forward(full[r], dim=1), torch.cat(full, dim=1))
# receive straight into the tail of a joint [text; image] buffer (Qwen block) and gather replicated text heads
joint = torch.zeros(2 + P * 6, 3, 4 // P, 8)
distribute.heads_to_sequence(qkv[r].clone(), out=joint[2:])
assert torch.equal(joint[2:], exp) and bool((joint[:2] == 0).all()), "heads_to_sequence(out=)"
txt = torch.randn(5, 4, 8, generator=g)                                   # replicated on every rank
got_txt = distribute.gather_heads(txt[:, r * (4 // P):(r + 1) * (4 // P)].contiguous())
assert torch.equal(got_txt, txt), "gather_heads"
dist.barrier(); dist.destroy_process_group()
print("rank", r, "ok")
"""


def test_ulysses_exchange_world_size_2_gloo(tmp_path):
    script = tmp_path / "a2a_worker.py"
    script.write_text(_A2A_WORKER)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29541")
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    for p in procs:
        out, _ = p.communicate(timeout=120)
        assert p.returncode == 0, out.decode()


def test_install_registers_into_ksana_when_present():
    """Runs only where the KsanaDiT tree is importable (the development container)."""
    ref = os.environ.get("KSANA_REFERENCE", "/root/reference")
    if not os.path.isdir(os.path.join(ref, "ksana")):
        pytest.skip("KsanaDiT source tree not present")
    code = f"""
import sys
sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {os.path.join(ROOT, 'tests', 'golden')!r})
import make_golden; make_golden.install_stubs()
import ksana
from ksana.config import KsanaAttentionBackend, KsanaAttentionConfig
from ksana.operations.attention.backends import base
from ksanadit_b200 import install, attention, linear
install.install()
m = base.get_backend_mapping()
assert issubclass(m[KsanaAttentionBackend.SAGE_ATTN], attention.B200SageAttentionImpl)
assert issubclass(m[KsanaAttentionBackend.SAGE_ATTN], base.KsanaAttentionBackendImpl)
assert m[KsanaAttentionBackend.RADIAL_SAGE_ATTN].type() == KsanaAttentionBackend.RADIAL_SAGE_ATTN
import torch, ksana.operations.ops as ops_mod
cls = ops_mod.pick_linear(torch.bfloat16, {{"w": torch.zeros(2,2).to(torch.float8_e4m3fn)}}, "default", None)
assert issubclass(cls, linear.B200Fp8Linear)
import ksana.operations.fuse_qkv.fuse_qkv as fq
class O: Linear = cls
assert fq.should_use_qkv_fusion(O) is True
install.uninstall()
assert not issubclass(base.get_backend_mapping()[KsanaAttentionBackend.SAGE_ATTN], attention.B200SageAttentionImpl)
print("install ok")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "install ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_torch_library_ops_have_shape_inference():
    """The registered operators can be traced with fake tensors (no kernel runs) and refuse CPU tensors."""
    import pytest
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode

    import ksanadit_b200.torch_ops  # noqa: F401  (registers torch.ops.ksana_b200.*)
    with FakeTensorMode():
        x = torch.empty(2, 7, 64, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(48, 64, dtype=torch.float8_e4m3fn, device="cuda")
        s = torch.empty(48, dtype=torch.float32, device="cuda")
        y = torch.ops.ksana_b200.fp8_linear(x, w, s, None)
        assert y.shape == (2, 7, 48) and y.dtype == torch.bfloat16
        q = torch.empty(100, 4, 128, dtype=torch.float16, device="cuda")
        o = torch.ops.ksana_b200.sage_attention(q, q, q)
        assert o.shape == q.shape and o.dtype == torch.float16
    with pytest.raises(Exception):
        torch.ops.ksana_b200.sage_attention(torch.zeros(8, 1, 128, dtype=torch.bfloat16), torch.zeros(8, 1, 128, dtype=torch.bfloat16),
                                            torch.zeros(8, 1, 128, dtype=torch.bfloat16))


def test_install_fused_blocks_adopts_the_reference_block():
    """Runs only where the KsanaDiT tree is importable: a WanAttentionBlock built from the installed operators is taken
    over by the fused sequence on its own parameters, its state dict is untouched, and uninstall restores the forward."""
    ref = os.environ.get("KSANA_REFERENCE", "/root/reference")
    if not os.path.isdir(os.path.join(ref, "ksana")):
        pytest.skip("KsanaDiT source tree not present")
    code = f"""
import sys
sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {os.path.join(ROOT, 'tests', 'golden')!r})
import make_golden; make_golden.install_stubs()
import torch, ksana
from ksana.config import KsanaAttentionBackend, KsanaAttentionConfig
from ksanadit_b200 import install, adopt, linear
install.install(fused_blocks=True)
from ksana.models.wan.wan_model import WanAttentionBlock
from ksana.operations.ops import LayerNorm, Ops, RMSNorm
from ksana.operations.linear.linear import Linear
from ksana.operations.attention.pick_attn import pick_attn_op
def build(lin, backend):
    ops = Ops()
    for n, c in (("Linear", lin), ("LayerNorm", LayerNorm), ("RMSNorm", RMSNorm)):
        ops.register(n, c)
    ops.register("Attn", pick_attn_op(KsanaAttentionConfig(backend=backend)))
    st = {{"operations": ops, "device": "cpu", "dtype": torch.bfloat16, "rms_dtype": None}}
    return WanAttentionBlock(256, 512, 2, block_id=3, qk_norm=True, cross_attn_norm=True, eps=1e-6, operation_settings=st)
blk = build(linear.b200_fp8_ops(scale_input=False), KsanaAttentionBackend.SAGE_ATTN)
keys = sorted(blk.state_dict())
assert adopt.why_not_adoptable(blk) is None
ab = adopt.adopt(blk)
assert ab is adopt.adopt(blk) and ab.block_id == 3 and ab.dtype == torch.bfloat16
assert ab.self_attn.qkv is blk.self_attn.qkv and ab.cross_attn.o is blk.cross_attn.o and ab.ffn[2] is blk.ffn[2]
assert ab.modulation is blk.modulation and ab.norm3 is blk.norm3
assert sorted(blk.state_dict()) == keys and not any(p is None for p in blk.parameters())
assert WanAttentionBlock.forward.__name__ == "fused_wan_forward"
# blocks that do not qualify keep their own forward: plain Linears, or another attention backend
assert "separate Linears" in adopt.why_not_adoptable(build(Linear, KsanaAttentionBackend.SAGE_ATTN))
assert "Sage" in adopt.why_not_adoptable(build(linear.b200_fp8_ops(), KsanaAttentionBackend.TORCH_SDPA))
plain = build(Linear, KsanaAttentionBackend.TORCH_SDPA)
from ksana.operations.attention.backends.sdpa import SDPAImpl
SDPAImpl.supports = staticmethod(lambda **_: True)
from ksana.models.wan.wan_model import rope_params
freqs = torch.cat([rope_params(1024, 44), rope_params(1024, 42), rope_params(1024, 42)], dim=1)
for p_ in plain.parameters():
    torch.nn.init.normal_(p_, std=0.02)
x = torch.randn(1, 24, 256).to(torch.bfloat16); e = torch.randn(1, 1, 6, 256).to(torch.bfloat16); c = torch.randn(1, 8, 256).to(torch.bfloat16)
with torch.no_grad():
    y = plain(x, e, seq_lens=torch.tensor([24]), grid_sizes=torch.tensor([[2, 3, 4]]), freqs=freqs, context=c, context_lens=None,
              step_iter=0, latent_shape=[1, 16, 2, 6, 8])
install.uninstall()
assert WanAttentionBlock.forward.__name__ == "forward"
with torch.no_grad():
    y2 = plain(x, e, seq_lens=torch.tensor([24]), grid_sizes=torch.tensor([[2, 3, 4]]), freqs=freqs, context=c, context_lens=None,
               step_iter=0, latent_shape=[1, 16, 2, 6, 8])
assert torch.equal(y, y2)  # the patched forward handed the non-qualifying block to the original one
# the Qwen-Image dual-stream block is adopted the same way
install.install(fused_blocks=True)
from ksana.models.qwen.transformer import QwenImageTransformerBlock
ops = Ops()
for n, c in (("Linear", linear.b200_fp8_ops()), ("LayerNorm", LayerNorm), ("RMSNorm", RMSNorm)):
    ops.register(n, c)
ops.register("Attn", pick_attn_op(KsanaAttentionConfig(backend=KsanaAttentionBackend.SAGE_ATTN)))
qb = QwenImageTransformerBlock(256, 2, 128, operation_settings={{"operations": ops, "device": "cpu", "dtype": torch.bfloat16, "rms_dtype": None}})
qkeys = sorted(qb.state_dict())
assert adopt.why_not_adoptable_qwen(qb) is None
qa = adopt.adopt_qwen(qb)
assert qa.attn.to_qkv is qb.attn.to_qkv and qa.txt_mlp.net[2] is qb.txt_mlp.net[2] and qa.img_mod[1] is qb.img_mod[1]
assert qa._norm_weight("norm_added_k").dtype == torch.float32 and sorted(qb.state_dict()) == qkeys
assert QwenImageTransformerBlock.forward.__name__ == "fused_qwen_forward"
install.uninstall()
assert QwenImageTransformerBlock.forward.__name__ == "forward"
print("adopt ok")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "adopt ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_pair_tile_lists_are_the_unions_of_the_block_lists():
    """radial_mask.pair_tile_lists: per pair of Q blocks the union of the two lists in ascending tile order, each entry
    carrying both blocks' keep bits; odd block counts (last pair = one block), empty lists, an all-empty mask."""
    import numpy as np

    from ksanadit_b200 import radial_mask as PM
    rng = np.random.RandomState(0)
    for nq, nk64, density in [(1, 2, 0.5), (3, 7, 0.4), (8, 16, 0.4), (5, 9, 0.1), (4, 6, 0.0)]:
        m = rng.random_sample((nq, nk64)) < density
        o, e = PM.compact_tile_lists(m)
        po, pe = PM.pair_tile_lists(o, e)
        assert po.dtype == np.int32 and pe.dtype == np.int32 and po.size == (nq + 1) // 2 + 1 and po[-1] == pe.size
        for pr in range((nq + 1) // 2):
            want = {}
            for b in (0, 1):
                q = 2 * pr + b
                if q < nq:
                    for ent in e[o[q]:o[q + 1]]:
                        want[int(ent) >> 2] = want.get(int(ent) >> 2, 0) | ((int(ent) & 3) << (2 * b))
            got = pe[po[pr]:po[pr + 1]]
            assert [int(x) >> 4 for x in got] == sorted(want)
            assert {int(x) >> 4: int(x) & 15 for x in got} == want

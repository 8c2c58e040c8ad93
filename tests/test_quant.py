"""Weight quantisers: format definitions on CPU, native kernels against them on the GPU."""
import pytest
import torch

from axon_b200.ops import quant as Q


def _w(M, N, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(M, N, generator=g) * torch.rand(M, 1, generator=g) * 3
    w[0, :min(128, N)] = 0
    return w.to(torch.bfloat16).to(device)


def test_int4_format_roundtrip():
    w = _w(16, 256)
    q, s = Q.int4_group_quant_ref(w, 128)
    assert q.min() >= -8 and q.max() <= 7 and s.shape == (16, 2)
    packed = Q.pack_int4_to_int32(q)
    assert packed.dtype == torch.int32 and packed.shape == (16, 32)
    assert torch.equal(Q.unpack_int32_to_int4(packed), q)
    first = int(packed[1, 0].item()) & 0xFFFFFFFF
    assert [(first >> (4 * i)) & 0xF for i in range(8)] == [int(v) + 8 for v in q[1, :8]]
    deq = Q.int4_dequant(packed, s, 128)
    err = (deq - w.float()).abs().reshape(16, 2, 128).amax(-1)
    assert (err <= s.float() * 0.5 + 1e-2 * s.float()).all()
    assert (s[0, 0].float() - 1e-5).abs() < 1e-6                      # all-zero group: the scale floor


def test_mxfp8_format():
    w = _w(8, 128, seed=1)
    q, s = Q.mxfp8_quant_ref(w)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.uint8 and s.shape == (8, 4)
    deq = Q.mxfp8_dequant(q, s)
    rel = (deq - w.float()).abs() / w.float().abs().clamp_min(1e-3)
    assert rel[w.float().abs() > 0.05].max() < 0.07                   # e4m3: 3 mantissa bits
    scale = torch.exp2(s.float() - 127)
    amax = w.float().reshape(8, 4, 32).abs().amax(-1)
    live = amax > 0
    assert (amax[live] / scale[live] <= 448).all() and (amax[live] / scale[live] > 224).all()
    assert s[0, 0] == 0 and s[0, 1] == 0                              # zero groups: smallest scale


def test_fp8_block_roundtrip():
    w = _w(200, 300, seed=2)
    q, s = Q.fp8_block_quant(w)
    assert s.shape == (2, 3)
    deq = Q.fp8_block_dequant(q, s)
    assert ((deq - w.float()).abs() <= w.float().abs() * 0.07 + s.max() * 0.6).all()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,group", [(64, 4096, 128), (33, 512, 32), (128, 1024, 64)])
def test_int4_kernel_matches_reference(M, N, group):
    w = _w(M, N, seed=3, device="cuda")
    packed, scales = Q.int4_quant_pack(w, group)
    q_ref, s_ref = Q.int4_group_quant_ref(w, group)
    assert torch.equal(scales, s_ref)
    assert torch.equal(packed, Q.pack_int4_to_int32(q_ref))


@pytest.mark.gpu
@pytest.mark.parametrize("M,N", [(64, 4096), (7, 96)])
def test_mxfp8_kernel_matches_reference(M, N):
    w = _w(M, N, seed=4, device="cuda")
    q, s = Q.mxfp8_quant(w)
    q_ref, s_ref = Q.mxfp8_quant_ref(w)
    assert torch.equal(s, s_ref)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))


@pytest.mark.gpu
def test_fp8_block_kernel_matches_reference():
    from axon_b200.utils.p2p.plan import fp8_block_quant_ref
    w = _w(384, 640, seed=5, device="cuda")
    q, s = Q.fp8_block_quant(w)
    q_ref, s_ref = fp8_block_quant_ref(w)
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3     # ties at rounding boundaries


def test_quantizing_generators_names_and_filters():
    from axon_b200.utils.quant import quantize_weights, should_quantize_param
    assert should_quantize_param("model.layers.0.self_attn.q_proj.weight")
    assert should_quantize_param("model.layers.3.mlp.experts.7.down_proj.weight")
    for bad in ("model.embed_tokens.weight", "lm_head.weight", "model.layers.0.input_layernorm.weight",
                "model.layers.0.mlp.gate.weight", "model.layers.0.self_attn.q_proj.bias", "model.norm.weight"):
        assert not should_quantize_param(bad), bad
    w = {"model.layers.0.self_attn.q_proj.weight": _w(256, 256), "model.layers.0.input_layernorm.weight": torch.ones(256),
         "model.layers.0.mlp.down_proj.weight": _w(256, 384, seed=9), "lm_head.weight": _w(64, 256)}
    out = dict(quantize_weights(w.items(), "fp8"))
    assert out["model.layers.0.self_attn.q_proj.weight"].dtype == torch.float8_e4m3fn
    assert out["model.layers.0.self_attn.q_proj.weight_scale_inv"].shape == (2, 2)
    assert out["lm_head.weight"].dtype == torch.bfloat16 and "lm_head.weight_scale_inv" not in out
    out = dict(quantize_weights(w.items(), "int4", group_size=128, ignore=["model.layers.0.mlp.down_proj"]))
    assert out["model.layers.0.self_attn.q_proj.weight_packed"].shape == (256, 32)
    assert out["model.layers.0.self_attn.q_proj.weight_shape"].tolist() == [256, 256]
    assert "model.layers.0.mlp.down_proj.weight" in out and "model.layers.0.mlp.down_proj.weight_packed" not in out
    out = dict(quantize_weights(w.items(), "mxfp8"))
    assert out["model.layers.0.mlp.down_proj.weight_scale_inv"].shape == (256, 12)
    assert list(dict(quantize_weights(w.items(), None))) == list(w)
    with pytest.raises(ValueError):
        list(quantize_weights(w.items(), "int2"))

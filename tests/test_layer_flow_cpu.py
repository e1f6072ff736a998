"""The decoder layer's control flow on the CPU: every combination of its
options runs end to end against the fp32 reference, with the GPU kernels
replaced by host stand-ins that follow the kernels' contracts (the GEMM by a
plain fp32 product, the glue ops by the C++ oracles, the SwiGLU epilogue by the
tile layout it is defined on).  What this pins down is the plumbing between
the ops: shapes, buffers, weight interleaving, in-place semantics, residuals.
"""
import pytest
import torch

from symm_mem_recipes_b200._ext import C as REAL_C


class _FakeC:
    """Host stand-ins with the signatures of the native entry points the layer reaches."""

    def __getattr__(self, name):
        return getattr(REAL_C, name)

    @staticmethod
    def ag_matmul(a, b, c, mode, aout_alloc, aout_offset, a_out, block_n, num_sms, timeout_ns, tail_scratch=None,
                  epilogue=0, trace=None, lead=-1, push_ahead=0, push_plain_stores=False,
                  push_pieces=0, panel_w=0):
        assert mode == 0, "world of one: no gather"
        full = a.float() @ b.float().t()
        if epilogue == 1:
            assert block_n == 256 and full.shape[1] % 256 == 0
            tiles = full.view(full.shape[0], -1, 2, 128)                 # [M, tile, gate|up, 128]
            full = (torch.nn.functional.silu(tiles[:, :, 0]) * tiles[:, :, 1]).reshape(full.shape[0], -1)
        assert tuple(c.shape) == tuple(full.shape)
        c.copy_(full.to(c.dtype))

    @staticmethod
    def rms_norm(x, residual, w, sum_out, out, eps):
        o, s = REAL_C.oracle_rms_norm_bf16(x, residual, w, eps)
        out.copy_(o)
        if sum_out is not None:
            sum_out.copy_(s)

    @staticmethod
    def rope_inplace(qkv, n_heads, head_dim, seq, pos0, theta, num_sms, pos=None):
        pos0 = pos0 if pos is None else int(pos)
        qkv.copy_(REAL_C.oracle_rope_bf16(qkv, n_heads, head_dim, seq, pos0, theta))

    @staticmethod
    def decode_attention(qkv, k_cache, v_cache, out, scratch, hq, hkv, pos0, pos=None, rope_theta=0.0):
        where = pos0 if pos is None else int(pos)
        if rope_theta:
            qkv = REAL_C.oracle_rope_bf16(qkv, hq + hkv, k_cache.shape[3], 1, where, rope_theta)
        out.copy_(REAL_C.oracle_decode_attention_bf16(qkv, k_cache, v_cache, hq, hkv, where))

    @staticmethod
    def silu_mul(gate_up, out, num_sms):
        out.copy_(REAL_C.oracle_silu_mul_bf16(gate_up))


@pytest.fixture
def host_kernels(monkeypatch):
    from symm_mem_recipes_b200.ops import ag_matmul, layer_glue

    fake = _FakeC()
    for mod in (ag_matmul, layer_glue):
        monkeypatch.setattr(mod, "C", fake)
    monkeypatch.setattr(ag_matmul, "_num_sms", lambda device: 148)
    monkeypatch.setattr(layer_glue, "_num_sms", lambda device: 148)
    monkeypatch.setattr(ag_matmul, "_tail_buffer", lambda device, config: None)

    def relaxed_2d(name, t, dtype=None):
        assert t.dim() == 2 and t.is_contiguous(), name
        assert dtype is None or t.dtype == dtype, name

    def relaxed(name, t, dim):
        assert t.dim() == dim and t.is_contiguous() and t.dtype == torch.bfloat16, name

    monkeypatch.setattr(ag_matmul, "_check_2d", relaxed_2d)
    monkeypatch.setattr(layer_glue, "_check", relaxed)


def _layer_and_reference(fused_glue, fused_swiglu, **kw):
    from symm_mem_recipes_b200.models.llama_tp_layer import (LlamaTPConfig, LlamaTPDecoderLayer,
                                                             full_precision_reference)

    cfg = LlamaTPConfig.tiny(1)
    layer = LlamaTPDecoderLayer(cfg, torch.device("cpu"), seed=1, fused_glue=fused_glue, fused_swiglu=fused_swiglu,
                                **kw)
    batch, seq = 2, 16
    torch.manual_seed(3)
    x = (torch.randn(batch * seq, cfg.hidden) * 0.5).to(torch.bfloat16)
    weights = [(layer.w_qkv, layer.w_o, layer.w_gate_up, layer.w_down, layer.norm1, layer.norm2)]
    ref = full_precision_reference(weights, cfg, x, batch, seq)
    return cfg, layer, x, batch, seq, ref


@pytest.mark.parametrize("fused_glue,fused_swiglu", [(False, False), (True, False), (True, True), (False, True)])
def test_prefill_flow_matches_fp32(host_kernels, fused_glue, fused_swiglu):
    cfg, layer, x, batch, seq, ref = _layer_and_reference(fused_glue, fused_swiglu)
    x_before = x.clone()
    y = layer.forward(x, batch, seq)
    assert y.shape == x.shape and torch.equal(x, x_before)          # the input is not modified
    assert (y.float() - ref).abs().max().item() < 0.1
    y2 = layer.forward(x, batch, seq)                                # buffers are reused: same result again
    assert torch.equal(y, y2)
    y3 = layer.forward(x, batch, seq, barrier_between_phases=True)   # the optional phase barriers change nothing
    assert torch.equal(y, y3)
    y_lib = layer.forward_reference(x, batch, seq)
    assert (y.float() - y_lib.float()).abs().max().item() < 0.1


@pytest.mark.parametrize("fused_glue,shared", [(False, False), (True, False), (True, True)])
def test_decode_flow_matches_prefill(host_kernels, fused_glue, shared):
    """Decoding the tokens one by one through the KV cache gives what the
    prefill of the same sequence gives at every position."""
    cfg, layer, x, batch, seq, _ = _layer_and_reference(fused_glue, False, shared_row_weights=shared)
    assert (layer.w_o_t is None) == shared                        # one copy of the row-parallel weights
    want = layer.forward(x, batch, seq).view(batch, seq, cfg.hidden)
    k_cache = torch.zeros(batch, seq, layer.hkv, cfg.head_dim, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    xs = x.view(batch, seq, cfg.hidden)
    for pos in range(seq):
        got = layer.decode(xs[:, pos].contiguous(), k_cache, v_cache, pos, fused=True)
        assert (got.float() - want[:, pos].float()).abs().max().item() < 0.1, pos


@pytest.mark.parametrize("fused_glue", [False, True])
def test_static_decode_matches_decode(host_kernels, fused_glue):
    """The graph-capturable form (position in a tensor, whole-cache attention
    under a mask, index_copy_ into the caches) against the plain decode step,
    token by token, with a cache longer than the sequence."""
    cfg, layer, x, batch, seq, _ = _layer_and_reference(fused_glue, False)
    xs = x.view(batch, seq, cfg.hidden)
    caches = [torch.zeros(batch, s_max, layer.hkv, cfg.head_dim, dtype=torch.bfloat16)
              for s_max in (seq, seq, seq + 5, seq + 5)]
    (k_a, v_a, k_b, v_b) = caches
    k_b.fill_(7.0)                                     # stale entries beyond the position must stay hidden
    v_b.fill_(-3.0)
    pos_t = torch.zeros(1, dtype=torch.int32)
    for pos in range(seq):
        step_in = xs[:, pos].contiguous()
        want = layer.decode(step_in, k_a, v_a, pos, fused=True)
        pos_t.fill_(pos)
        got = layer.decode_static(step_in, k_b, v_b, pos_t, fused=True)
        assert (got.float() - want.float()).abs().max().item() < 2e-2, pos
    assert torch.equal(k_b[:, :seq], k_a) and torch.equal(v_b[:, :seq], v_a)
    assert bool((k_b[:, seq:] == 7.0).all()) and bool((v_b[:, seq:] == -3.0).all())


@pytest.mark.parametrize("fused_glue,tp", [(False, False), (True, False), (True, True)])
def test_prefill_hands_its_kv_cache_to_decode(host_kernels, fused_glue, tp):
    """Prefill of a prompt that also fills the KV cache, then decode of the following tokens:
    same outputs as the prefill of the whole sequence, and the same cache as decoding all the way."""
    cfg, layer, x, batch, seq, _ = _layer_and_reference(fused_glue, False)
    prompt = seq // 2
    xs = x.view(batch, seq, cfg.hidden)
    want = layer.forward(x, batch, seq).view(batch, seq, cfg.hidden)
    k_cache = torch.zeros(batch, seq + 3, layer.hkv, cfg.head_dim, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    x_prompt = xs[:, :prompt].reshape(batch * prompt, cfg.hidden).contiguous()
    fwd = layer.forward_tp if tp else layer.forward
    y_prompt = fwd(x_prompt, batch, prompt, kv_cache=(k_cache, v_cache)).view(batch, prompt, cfg.hidden)
    assert (y_prompt.float() - want[:, :prompt].float()).abs().max().item() < 0.1
    for pos in range(prompt, seq):
        got = layer.decode(xs[:, pos].contiguous(), k_cache, v_cache, pos, fused=True)
        assert (got.float() - want[:, pos].float()).abs().max().item() < 0.1, pos
    # the cache a token-by-token decode builds is the same
    k2, v2 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    for pos in range(seq):
        layer.decode(xs[:, pos].contiguous(), k2, v2, pos, fused=True)
    assert (k_cache.float() - k2.float()).abs().max().item() < 0.05
    assert (v_cache.float() - v2.float()).abs().max().item() < 0.05
    with pytest.raises(ValueError, match="kv_cache"):
        layer.forward(x, batch, seq, kv_cache=(k_cache[:, :4], v_cache[:, :4]))


def test_stack_prefill_then_decode(host_kernels):
    """Two layers as a serving loop drives them: prefill of the prompt, then token-by-token decode;
    against the prefill of the whole sequence through the same two layers."""
    from symm_mem_recipes_b200.models.llama_tp_layer import LlamaTPConfig, LlamaTPStack

    cfg = LlamaTPConfig.tiny(1)
    batch, seq, prompt = 2, 24, 16
    stack = LlamaTPStack(cfg, 2, torch.device("cpu"), batch, max_seq=seq + 4, seed=5, fused_glue=True)
    assert stack.graph is None and len(stack.caches) == 2                  # no CUDA graphs on the CPU
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(batch, seq, cfg.hidden, generator=g) * 0.5).to(torch.bfloat16)
    whole = x.reshape(batch * seq, cfg.hidden)
    for lyr in stack.layers:
        whole = lyr.forward(whole, batch, seq)
    whole = whole.view(batch, seq, cfg.hidden)
    y_prompt = stack.prefill(x[:, :prompt].reshape(batch * prompt, cfg.hidden).contiguous(), prompt)
    assert (y_prompt.view(batch, prompt, -1).float() - whole[:, :prompt].float()).abs().max().item() < 0.1
    for pos in range(prompt, seq):
        y = stack.decode_step(x[:, pos].contiguous(), pos)
        assert (y.float() - whole[:, pos].float()).abs().max().item() < 0.15, pos
    with pytest.raises(ValueError, match="outside the cache"):
        stack.decode_step(x[:, 0].contiguous(), seq + 4)
    stack.reset()
    assert float(stack.caches[0][0].abs().sum()) == 0.0


def test_residual_chaining_between_layers_changes_no_bit(host_kernels):
    """x1 + down of one layer computed by the next layer's first RMSNorm kernel: same bits as the
    separate add, and layers without the glue kernels are left out of the chain."""
    from symm_mem_recipes_b200.models.llama_tp_layer import (LlamaTPConfig, LlamaTPDecoderLayer,
                                                              decode_static_through, new_kv_caches)

    cfg = LlamaTPConfig.tiny(1)
    dev = torch.device("cpu")
    glue = [True, True, False, True]
    layers = [LlamaTPDecoderLayer(cfg, dev, seed=7 + i, fused_glue=g) for i, g in enumerate(glue)]
    assert [lyr.chains_residual() for lyr in layers] == glue
    a, b = new_kv_caches(layers, 2, 8), new_kv_caches(layers, 2, 8)
    pos = torch.zeros(1, dtype=torch.int32)
    g = torch.Generator().manual_seed(1)
    for step in range(3):
        x = (torch.randn(2, cfg.hidden, generator=g) * 0.5).to(torch.bfloat16)
        pos.fill_(step)
        chained = decode_static_through(layers, a, x, pos)
        plain = x
        for lyr, (kc, vc) in zip(layers, b):
            plain = lyr.decode_static(plain, kc, vc, pos)
        assert torch.equal(chained, plain), step
    with pytest.raises(ValueError, match="glue kernels"):
        layers[2].decode_static(x, *b[2], pos, defer_residual=True)


def test_phase_marks_are_off_by_default(host_kernels):
    _, layer, x, batch, seq, _ = _layer_and_reference(False, False)
    layer.forward(x, batch, seq)
    assert layer.phase_marks is None


@pytest.mark.parametrize("fused_glue,fused_swiglu", [(False, False), (True, False), (True, True)])
def test_tensor_parallel_prefill_flow_matches_fp32(host_kernels, fused_glue, fused_swiglu):
    """Without sequence parallelism (replicated activations, all-reduce endings): same layer, same answer."""
    cfg, layer, x, batch, seq, ref = _layer_and_reference(fused_glue, fused_swiglu)
    y = layer.forward_tp(x, batch, seq)
    assert y.shape == x.shape and (y.float() - ref).abs().max().item() < 0.1
    y_lib = layer.forward_tp_reference(x, batch, seq)
    assert (y.float() - y_lib.float()).abs().max().item() < 0.1
    assert (y.float() - layer.forward(x, batch, seq).float()).abs().max().item() < 0.1

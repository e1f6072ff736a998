"""The TP decoder layer: fused forward vs the NCCL + cuBLAS forward vs fp32."""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import spawn_ranks


def _layer_worker(rank, world_size):
    from symm_mem_recipes_b200.models.llama_tp_layer import (LlamaTPConfig, LlamaTPDecoderLayer,
                                                              full_precision_reference)
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    cfg = LlamaTPConfig.tiny(world_size)
    layer = LlamaTPDecoderLayer(cfg, dev, seed=11)
    batch, seq = 2, 128 * world_size
    rows = batch * seq // world_size
    g = torch.Generator().manual_seed(5)
    x_full = (torch.randn(batch * seq, cfg.hidden, generator=g) * 0.5).to(torch.bfloat16)
    x_shard = x_full[rank * rows:(rank + 1) * rows].to(dev)
    failures = []
    y = layer.forward(x_shard, batch, seq, barrier_between_phases=True)
    symm_mem.check_status(dev)
    y_lib = layer.forward_reference(x_shard, batch, seq)
    if not torch.allclose(y.float(), y_lib.float(), rtol=5e-2, atol=5e-2):
        failures.append(f"fused vs NCCL+cuBLAS: {(y.float() - y_lib.float()).abs().max().item()}")
    # fp32 reference from every rank's weights (regenerated from their seeds on the CPU)
    weights = []
    for r in range(world_size):
        gw = torch.Generator().manual_seed(11 + r)
        H, D = cfg.hidden, cfg.head_dim

        def w(*shape):
            return (torch.randn(*shape, generator=gw) * 0.02).to(torch.bfloat16)

        w_qkv = w((layer.hq + 2 * layer.hkv) * D, H)
        w_o = w(H, layer.hq * D)
        w_gu = w(2 * layer.ffn_local, H)
        w_down = w(H, layer.ffn_local)
        weights.append((w_qkv, w_o, w_gu, w_down, layer.norm1.cpu(), layer.norm2.cpu()))
    if not torch.equal(weights[rank][0], layer.w_qkv.cpu()):
        failures.append("weight regeneration does not match")
    ref = full_precision_reference(weights, cfg, x_full, batch, seq)[rank * rows:(rank + 1) * rows]
    err = (y.float().cpu() - ref).abs().max().item()
    if err > 0.1:
        failures.append(f"fused vs fp32 reference: {err}")

    # decode: fused GEMV + all-reduce vs cuBLAS + NCCL
    B, smax = 4, 16
    xd = (torch.randn(B, cfg.hidden, generator=torch.Generator().manual_seed(9)) * 0.5).to(torch.bfloat16).to(dev)
    kc = torch.zeros(B, smax, layer.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    for pos in range(3):
        yd = layer.decode(xd, kc, vc, pos, fused=True)
        yr = layer.decode(xd, kc2, vc2, pos, fused=False)
        symm_mem.check_status(dev)
        if not torch.allclose(yd.float(), yr.float(), rtol=5e-2, atol=5e-2):
            failures.append(f"decode pos {pos}: {(yd.float() - yr.float()).abs().max().item()}")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
def test_layer_world_of_one():
    from symm_mem_recipes_b200.models.llama_tp_layer import smoke

    torch.cuda.set_device(0)
    smoke(torch.device("cuda", 0))


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_layer_2gpu():
    spawn_ranks(_layer_worker, 2, "nccl")


@pytest.mark.gpu
@pytest.mark.multigpu(4)
def test_layer_4gpu():
    spawn_ranks(_layer_worker, 4, "nccl")


def _layer_tp_worker(rank, world_size, fused_glue, fused_swiglu):
    """Prefill without sequence parallelism (matmul_all_reduce endings) and the sequence-parallel
    prefill with the single-pass glue kernels, against the library compositions."""
    from symm_mem_recipes_b200.models.llama_tp_layer import LlamaTPConfig, LlamaTPDecoderLayer
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    cfg = LlamaTPConfig.tiny(world_size)
    layer = LlamaTPDecoderLayer(cfg, dev, seed=11, fused_glue=fused_glue, fused_swiglu=fused_swiglu)
    batch, seq = 2, 128 * world_size
    rows = batch * seq // world_size
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(batch * seq, cfg.hidden, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    failures = []
    for it in range(2):
        y_tp = layer.forward_tp(x, batch, seq)
        symm_mem.check_status(dev)
        y_tp_lib = layer.forward_tp_reference(x, batch, seq)
        if not torch.allclose(y_tp.float(), y_tp_lib.float(), rtol=5e-2, atol=5e-2):
            worst = (y_tp.float() - y_tp_lib.float()).abs().max().item()
            failures.append(f"call {it}: TP prefill vs cuBLAS + NCCL: {worst}")
        y_sp = layer.forward(x[rank * rows:(rank + 1) * rows].contiguous(), batch, seq)
        symm_mem.check_status(dev)
        if not torch.allclose(y_sp.float(), y_tp_lib[rank * rows:(rank + 1) * rows].float(), rtol=5e-2, atol=5e-2):
            failures.append(f"call {it}: SP prefill differs from the TP result")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("fused_glue,fused_swiglu", [(False, False), (True, True)])
def test_layer_tensor_parallel_prefill_2gpu(fused_glue, fused_swiglu):
    spawn_ranks(_layer_tp_worker, 2, "nccl", (fused_glue, fused_swiglu))


def _decode_graph_worker(rank, world_size, fused_glue):
    """Two layers, one captured graph, replayed for six positions: every step
    equals the eager decode step run beside it with its own caches."""
    from symm_mem_recipes_b200.models.llama_tp_layer import DecodeGraph, LlamaTPConfig, LlamaTPDecoderLayer
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    cfg = LlamaTPConfig.tiny(world_size)
    layers = [LlamaTPDecoderLayer(cfg, dev, seed=21 + 100 * i, fused_glue=fused_glue) for i in range(2)]
    batch, max_seq, steps = 4, 32, 6
    graph = DecodeGraph(layers, batch, max_seq)
    symm_mem.check_status(dev)
    eager_caches = [(torch.zeros(batch, max_seq, lyr.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev),
                     torch.zeros(batch, max_seq, lyr.hkv, cfg.head_dim, dtype=torch.bfloat16, device=dev))
                    for lyr in layers]
    g = torch.Generator().manual_seed(9)              # same tokens on every rank: activations are replicated
    failures = []
    for pos in range(steps):
        x = (torch.randn(batch, cfg.hidden, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        got = graph.step(x, pos).clone()
        want = x
        for lyr, (kc, vc) in zip(layers, eager_caches):
            want = lyr.decode(want, kc, vc, pos, fused=True)
        symm_mem.check_status(dev)
        err = (got.float() - want.float()).abs().max().item()
        if err > 5e-2:
            failures.append(f"position {pos}: graph replay differs from the eager step by {err}")
    for (kc, vc), (kg, vg) in zip(eager_caches, graph.caches):
        same_k = torch.allclose(kc.float(), kg.float(), atol=2e-2)
        if not (same_k and torch.allclose(vc.float(), vg.float(), atol=2e-2)):
            failures.append("KV caches of the graph differ from the eager ones")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
@pytest.mark.parametrize("fused_glue", [False, True])
def test_decode_graph_world_of_one(fused_glue):
    torch.cuda.set_device(0)
    _decode_graph_worker(0, 1, fused_glue)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("fused_glue", [False, True])
def test_decode_graph_2gpu(fused_glue):
    spawn_ranks(_decode_graph_worker, 2, "nccl", (fused_glue,))


def _stack_worker(rank, world_size):
    """LlamaTPStack as a serving loop drives it: sequence-parallel prefill of the prompt into the
    caches, then decode from the captured graph; against the prefill of the whole sequence."""
    from symm_mem_recipes_b200.models.llama_tp_layer import LlamaTPConfig, LlamaTPStack
    from symm_mem_recipes_b200.parallel import symm_mem

    dev = torch.device("cuda", rank)
    cfg = LlamaTPConfig.tiny(world_size)
    batch, prompt, new_tokens = 2, 64 * world_size, 4
    seq = prompt + new_tokens
    stack = LlamaTPStack(cfg, 2, dev, batch, max_seq=seq + 8, seed=5)
    assert stack.graph is not None
    g = torch.Generator().manual_seed(2)              # same activations on every rank
    x = (torch.randn(batch, seq, cfg.hidden, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    rows = batch * prompt // world_size
    x_prompt = x[:, :prompt].reshape(batch * prompt, cfg.hidden)
    y_prompt = stack.prefill(x_prompt[rank * rows:(rank + 1) * rows].contiguous(), prompt)
    symm_mem.check_status(dev)
    # reference: the library composition of the same layers, token by token through caches of its own
    ref_caches = [(torch.zeros_like(kc), torch.zeros_like(vc)) for kc, vc in stack.caches]
    failures = []
    ref_prompt = x_prompt[rank * rows:(rank + 1) * rows].contiguous()
    for lyr in stack.layers:
        ref_prompt = lyr.forward_reference(ref_prompt, batch, prompt)
    if not torch.allclose(y_prompt.float(), ref_prompt.float(), rtol=5e-2, atol=5e-2):
        failures.append("prefill differs from the library composition")
    for pos in range(seq):                            # fills the reference caches from position 0
        h = x[:, pos].contiguous()
        for lyr, (kc, vc) in zip(stack.layers, ref_caches):
            h = lyr.decode(h, kc, vc, pos, fused=False)
        if pos >= prompt:
            y = stack.decode_step(x[:, pos].contiguous(), pos).clone()
            symm_mem.check_status(dev)
            err = (y.float() - h.float()).abs().max().item()
            if err > 0.1:
                failures.append(f"position {pos}: decode after prefill differs from the library composition by {err}")
    torch.cuda.synchronize()
    assert not failures, failures


@pytest.mark.gpu
def test_stack_prefill_then_graph_decode_world_of_one():
    torch.cuda.set_device(0)
    _stack_worker(0, 1)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_stack_prefill_then_graph_decode_2gpu():
    spawn_ranks(_stack_worker, 2, "nccl")

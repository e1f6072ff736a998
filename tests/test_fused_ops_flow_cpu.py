"""Host-side plumbing of the fused multi-rank ops with gloo ranks: which
branch a call takes, which allocation and offset it hands to the kernel, the
geometry rule of the gather buffer, the ordinary-a_out path by push and copy,
the weight interleaving of the SwiGLU epilogue.  The kernels are replaced by
host stand-ins that move the same bytes through the POSIX-shm symmetric memory
(each rank writes its shard into every rank's a_out, as the push gather does).
"""
import pytest
import torch

from symm_mem_recipes_b200.utils.testing import spawn_ranks


def _install_host_kernels():
    import torch.distributed as dist

    from symm_mem_recipes_b200._ext import C as real
    from symm_mem_recipes_b200.ops import ag_matmul

    calls = []

    class Fake:
        def __getattr__(self, name):
            return getattr(real, name)

        @staticmethod
        def ag_matmul(a, b, c, mode, aout_alloc, aout_offset, a_out, block_n, num_sms, timeout_ns, tail_scratch=None,
                      epilogue=0, trace=None, lead=-1, push_ahead=0, push_plain_stores=False,
                      push_pieces=0, panel_w=0):
            calls.append(mode)
            if mode == 2:
                ws, rank = dist.get_world_size(), dist.get_rank()
                rows, K = a.shape
                assert a_out.data_ptr() == real.host_view(aout_alloc, -1, [1], torch.uint8, aout_offset).data_ptr()
                dist.barrier()                                   # the kernel's entry barrier
                for r in range(ws):                              # push: own shard into every rank's a_out
                    peer = real.host_view(aout_alloc, r, [rows * ws, K], a.dtype, aout_offset)
                    peer[rank * rows:(rank + 1) * rows].copy_(a)
                dist.barrier()                                   # arrival of every shard
                full_a = a_out
            else:
                assert mode == 0
                full_a = a
            full = full_a.float() @ b.float().t()
            if epilogue == 1:
                tiles = full.view(full.shape[0], -1, 2, 128)
                full = (torch.nn.functional.silu(tiles[:, :, 0]) * tiles[:, :, 1]).reshape(full.shape[0], -1)
            c.copy_(full.to(c.dtype))

    ag_matmul.C = Fake()
    ag_matmul._num_sms = lambda device: 148
    ag_matmul._tail_buffer = lambda device, config: None

    def relaxed_2d(name, t, dtype=None):
        assert t.dim() == 2 and t.is_contiguous(), name
        assert dtype is None or t.dtype == dtype, name

    ag_matmul._check_2d = relaxed_2d
    return calls


def _agmm_flow_worker(rank, world_size):
    import torch.distributed as dist

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200.errors import SymmMemError
    from symm_mem_recipes_b200.ops.ag_matmul import interleave_gate_up
    from symm_mem_recipes_b200.parallel import symm_mem

    calls = _install_host_kernels()
    rows, K, F = 128, 64, 256
    M = rows * world_size
    g = torch.Generator().manual_seed(5)
    wg = (torch.randn(F, K, generator=g) * 0.3).to(torch.bfloat16)
    wu = (torch.randn(F, K, generator=g) * 0.3).to(torch.bfloat16)
    shards = [(torch.randn(rows, K, generator=torch.Generator().manual_seed(10 + r)) * 0.5).to(torch.bfloat16)
              for r in range(world_size)]
    full_a = torch.cat(shards)
    a_shard = symm_mem.empty(rows, K, dtype=torch.bfloat16, device="cpu")
    a_shard.copy_(shards[rank])

    # 1. a_out = None: the internal symmetric buffer, gathered by push
    c = smr.all_gather_matmul(a_shard, wg)
    assert calls[-1] == 2 and c.shape == (M, F)
    assert torch.allclose(c.float(), full_a.float() @ wg.float().t(), atol=0.05)

    # 2. a symmetric a_out placed at an offset inside a larger allocation
    big = symm_mem.empty(2 * M * K, dtype=torch.bfloat16, device="cpu")
    a_out = big[M * K:].view(M, K)
    c2 = smr.all_gather_matmul(a_shard, wg, a_out)
    assert torch.equal(a_out, full_a) and torch.equal(c2, c)
    # the same allocation may not serve a gather of another geometry
    with pytest.raises(SymmMemError, match="already serves"):
        smr.all_gather_matmul(a_shard, wg, big[: M * K].view(M, K))
    dist.barrier()

    # 3. an ordinary a_out: gathered into the internal buffer, then one copy
    plain = torch.zeros(M, K, dtype=torch.bfloat16)
    c3 = smr.all_gather_matmul(a_shard, wg, plain)
    assert calls[-1] == 2 and torch.equal(plain, full_a) and torch.equal(c3, c)

    # 4. SwiGLU epilogue over the gather
    act = smr.all_gather_matmul(a_shard, interleave_gate_up(wg, wu), epilogue="swiglu")
    want = torch.nn.functional.silu(full_a.float() @ wg.float().t()) * (full_a.float() @ wu.float().t())
    assert act.shape == (M, F) and torch.allclose(act.float(), want, atol=0.05)

    # 5. mm_only: no communication, multiplies what it is given
    c5 = smr.all_gather_matmul(a_shard, wg, a_out=a_out, mm_only=True)
    assert calls[-1] == 0 and torch.equal(c5, c)

    # 6. shape errors are raised on the host
    with pytest.raises(SymmMemError, match="rows per rank"):
        smr.all_gather_matmul(a_shard[:100].contiguous(), wg)
    with pytest.raises(SymmMemError, match="a_out must be"):
        smr.all_gather_matmul(a_shard, wg, symm_mem.empty(M + 128, K, dtype=torch.bfloat16, device="cpu"))
    dist.barrier()


@pytest.mark.parametrize("world_size", [2, 4])
def test_all_gather_matmul_host_flow(world_size):
    spawn_ranks(_agmm_flow_worker, world_size, "gloo")


def _row_parallel_flow_worker(rank, world_size):
    import torch.distributed as dist

    import symm_mem_recipes_b200 as smr
    from symm_mem_recipes_b200._ext import C as real
    from symm_mem_recipes_b200.errors import SymmMemError
    from symm_mem_recipes_b200.parallel import symm_mem

    # the package re-exports functions under the names of these modules: import the modules themselves
    import importlib
    gemv_mod = importlib.import_module("symm_mem_recipes_b200.ops.gemv_all_reduce")
    rs_mod = importlib.import_module("symm_mem_recipes_b200.ops.matmul_reduce_scatter")
    seen = {}

    def summed(a, b):
        part = (a.float() @ b.float().t()).to(torch.bfloat16).float()     # bf16 partials, fp32 sum
        dist.all_reduce(part)
        return part

    class Fake:
        def __getattr__(self, name):
            return getattr(real, name)

        @staticmethod
        def matmul_reduce_scatter(a, b, out, workspace, num_sms, timeout_ns, trace=None, panel_w=0):
            seen["rs"] = workspace.payload_bytes
            rows = out.shape[0]
            out.copy_(summed(a, b)[rank * rows:(rank + 1) * rows].to(out.dtype))

        @staticmethod
        def matmul_all_reduce(a, b, out, out_alloc, out_offset, workspace, num_sms, timeout_ns, panel_w=0):
            assert out.data_ptr() == real.host_view(out_alloc, -1, [1], torch.uint8, out_offset).data_ptr()
            seen["ar"] = True
            out.copy_(summed(a, b).to(out.dtype))

        @staticmethod
        def gemv_all_reduce(x, w, out, workspace, ws_offset, timeout_ns, tensor_core=False, num_sms=148,
                            tagged=False, weights_nk=False):
            seen["gemv"] = (tensor_core, tagged)
            seen["gemv_nk"] = weights_nk
            part = x.float() @ (w.float().t() if weights_nk else w.float())
            dist.all_reduce(part)
            out.copy_(part.to(out.dtype))

    rs_mod.C = Fake()
    gemv_mod.C = Fake()
    rs_mod._num_sms = gemv_mod._num_sms = lambda device: 148

    M, N, K = 128 * world_size, 64, 32
    g = torch.Generator().manual_seed(100 + rank)
    a = (torch.randn(M, K, generator=g) * 0.3).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16)
    want = summed(a, b)
    rows = M // world_size

    out = smr.matmul_reduce_scatter(a, b)
    assert out.shape == (rows, N) and torch.allclose(out.float(), want[rank * rows:(rank + 1) * rows], atol=0.02)
    assert seen["rs"] >= real.matmul_rs_workspace_bytes(M, N)

    full = smr.matmul_all_reduce(a, b)                       # internal symmetric output, cached per shape
    assert symm_mem.is_symm_mem_tensor(full) and torch.allclose(full.float(), want, atol=0.02)
    assert smr.matmul_all_reduce(a, b).data_ptr() == full.data_ptr() and seen["ar"] is True
    with pytest.raises(SymmMemError, match="symmetric"):
        smr.matmul_all_reduce(a, b, out=torch.empty(M, N, dtype=torch.bfloat16))
    with pytest.raises(SymmMemError, match="multiple of 128"):
        smr.matmul_reduce_scatter(a[:100].contiguous(), b)

    x = (torch.randn(4, K, generator=g) * 0.3).to(torch.bfloat16)
    w = (torch.randn(K, N, generator=g) * 0.3).to(torch.bfloat16)
    y = smr.gemv_all_reduce(x, w)
    assert seen["gemv"] == (True, True) and y.shape == (4, N)                 # up to batch 8: the tagged exchange
    smr.gemv_all_reduce(torch.cat([x] * 4), w)
    assert seen["gemv"] == (True, False)                                       # batch 16: inboxes and flags
    smr.gemv_all_reduce(x, w, algo="tc")
    assert seen["gemv"] == (True, False)
    smr.gemv_all_reduce(x, w, algo="simt")
    assert seen["gemv"] == (False, False)
    y_nk = smr.gemv_all_reduce(x, w.t().contiguous(), weights_nk=True)       # [N, K] weights: same product
    assert seen["gemv_nk"] is True and torch.equal(y_nk, y)
    with pytest.raises(SymmMemError, match="tcgen05"):
        smr.gemv_all_reduce(x, w.t().contiguous(), algo="simt", weights_nk=True)
    ref = x.float() @ w.float()
    dist.all_reduce(ref)
    assert torch.allclose(y.float(), ref, atol=0.02)
    dist.barrier()


def test_row_parallel_ops_host_flow():
    spawn_ranks(_row_parallel_flow_worker, 2, "gloo")


def _install_row_parallel_and_glue_stand_ins():
    """matmul_reduce_scatter / matmul_all_reduce by a gloo all-reduce of bf16 partials, glue ops by the oracles."""
    import importlib

    import torch.distributed as dist

    from symm_mem_recipes_b200._ext import C as real

    rs_mod = importlib.import_module("symm_mem_recipes_b200.ops.matmul_reduce_scatter")
    glue_mod = importlib.import_module("symm_mem_recipes_b200.ops.layer_glue")

    def summed(a, b):
        part = (a.float() @ b.float().t()).to(torch.bfloat16).float()
        dist.all_reduce(part)
        return part

    class Fake:
        def __getattr__(self, name):
            return getattr(real, name)

        @staticmethod
        def matmul_reduce_scatter(a, b, out, workspace, num_sms, timeout_ns, trace=None, panel_w=0):
            rank, rows = dist.get_rank(), out.shape[0]
            out.copy_(summed(a, b)[rank * rows:(rank + 1) * rows].to(out.dtype))
            if trace is not None:                                # [CTA][start, entered, GEMM done, reduced] in ns
                trace.view(-1, 4)[:2] = torch.tensor([[1000, 2000, 9000, 12000], [1100, 2100, 9500, 12500]])

        @staticmethod
        def matmul_all_reduce(a, b, out, out_alloc, out_offset, workspace, num_sms, timeout_ns, panel_w=0):
            out.copy_(summed(a, b).to(out.dtype))

        @staticmethod
        def rms_norm(x, residual, w, sum_out, out, eps):
            o, s = real.oracle_rms_norm_bf16(x, residual, w, eps)
            out.copy_(o)
            if sum_out is not None:
                sum_out.copy_(s)

        @staticmethod
        def rope_inplace(qkv, n_heads, head_dim, seq, pos0, theta, num_sms, pos=None):
            pos0 = pos0 if pos is None else int(pos)
            qkv.copy_(real.oracle_rope_bf16(qkv, n_heads, head_dim, seq, pos0, theta))

        @staticmethod
        def decode_attention(qkv, k_cache, v_cache, out, scratch, hq, hkv, pos0, pos=None, rope_theta=0.0):
            where = pos0 if pos is None else int(pos)
            if rope_theta:
                qkv = real.oracle_rope_bf16(qkv, hq + hkv, k_cache.shape[3], 1, where, rope_theta)
            out.copy_(real.oracle_decode_attention_bf16(qkv, k_cache, v_cache, hq, hkv, where))

        @staticmethod
        def silu_mul(gate_up, out, num_sms):
            out.copy_(real.oracle_silu_mul_bf16(gate_up))

    rs_mod.C = glue_mod.C = Fake()
    rs_mod._num_sms = glue_mod._num_sms = lambda device: 148
    glue_mod._check = lambda name, t, dim: None


def _layer_flow_worker(rank, world_size, fused_glue, fused_swiglu):
    import torch.distributed as dist

    from symm_mem_recipes_b200.models.llama_tp_layer import (LlamaTPConfig, LlamaTPDecoderLayer,
                                                             full_precision_reference)

    _install_host_kernels()
    _install_row_parallel_and_glue_stand_ins()
    cfg = LlamaTPConfig.tiny(world_size)
    layer = LlamaTPDecoderLayer(cfg, torch.device("cpu"), seed=1, fused_glue=fused_glue, fused_swiglu=fused_swiglu)
    mine = (layer.w_qkv, layer.w_o, layer.w_gate_up, layer.w_down, layer.norm1, layer.norm2)
    weights = [None] * world_size
    dist.all_gather_object(weights, mine)
    batch, seq = 2, 64 * world_size                       # 128 token rows per rank
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(batch * seq, cfg.hidden, generator=g) * 0.5).to(torch.bfloat16)     # same on every rank
    ref = full_precision_reference(weights, cfg, x, batch, seq)
    rows = batch * seq // world_size

    # sequence-parallel prefill: token-sharded in, token-sharded out
    y = layer.forward(x[rank * rows:(rank + 1) * rows].contiguous(), batch, seq)
    assert (y.float() - ref[rank * rows:(rank + 1) * rows]).abs().max().item() < 0.15
    y_again = layer.forward(x[rank * rows:(rank + 1) * rows].contiguous(), batch, seq, barrier_between_phases=True)
    assert torch.equal(y, y_again)                        # the symmetric buffers are reused cleanly
    # plain tensor parallelism: replicated in, replicated out
    y_tp = layer.forward_tp(x, batch, seq)
    assert (y_tp.float() - ref).abs().max().item() < 0.15
    assert (y_tp[rank * rows:(rank + 1) * rows].float() - y.float()).abs().max().item() < 0.15
    # the library compositions agree too
    assert (layer.forward_tp_reference(x, batch, seq).float() - ref).abs().max().item() < 0.15
    dist.barrier()


@pytest.mark.parametrize("fused_glue,fused_swiglu", [(False, False), (True, True)])
def test_decoder_layer_host_flow_two_ranks(fused_glue, fused_swiglu):
    spawn_ranks(_layer_flow_worker, 2, "gloo", (fused_glue, fused_swiglu))


def _install_all_stand_ins():
    """Every kernel entry point the ops reach, as host code over gloo and the POSIX-shm symmetric
    memory; NCCL-only collectives of the library compositions re-expressed with what gloo has."""
    import importlib

    import torch.distributed as dist

    from symm_mem_recipes_b200._ext import C as real
    from symm_mem_recipes_b200.parallel import symm_mem

    _install_host_kernels()
    _install_row_parallel_and_glue_stand_ins()
    ag_mod = importlib.import_module("symm_mem_recipes_b200.ops.ag_matmul")
    gemv_mod = importlib.import_module("symm_mem_recipes_b200.ops.gemv_all_reduce")
    class GemvFake:
        def __getattr__(self, name):
            return getattr(real, name)

        @staticmethod
        def gemv_all_reduce(x, w, out, workspace, ws_offset, timeout_ns, tensor_core=False, num_sms=148, tagged=False,
                            weights_nk=False):
            part = x.float() @ (w.float().t() if weights_nk else w.float())
            dist.all_reduce(part)
            out.copy_(part.to(out.dtype))

    gemv_mod.C = GemvFake()
    gemv_mod._num_sms = lambda device: 148
    symm_mem.check_status = lambda device=None: None

    def reduce_scatter_by_all_reduce(out, inp, group=None):       # gloo has no reduce_scatter_tensor
        full = inp.float()
        dist.all_reduce(full, group=group)
        rows = out.shape[0]
        out.copy_(full[dist.get_rank() * rows:(dist.get_rank() + 1) * rows].to(out.dtype))

    dist.reduce_scatter_tensor = reduce_scatter_by_all_reduce


def _selfcheck_worker(rank, world_size):
    """The self-check program's own logic (shapes, references, outcome agreement) with host
    stand-ins for the kernels: a wrong reference there would cost GPU time to find."""
    import torch.distributed as dist

    from symm_mem_recipes_b200 import selfcheck

    _install_all_stand_ins()

    checks = [c for c in selfcheck.build_checks(world_size, rank, torch.device("cpu"))
              if not ((c[0] == "barrier" and "barrier" in c[1].lower()) or "NVLS" in c[1])]   # GPU-only kernels
    results, recoveries, stopped = selfcheck.run_checks(checks, rank, torch.device("cpu"))
    failures = [f"{r['group']}: {r['check']}: {r['detail']}" for r in results if not r["ok"]]
    assert not failures, failures
    assert len(results) >= 25 and recoveries == 0 and not stopped, (len(results), recoveries)
    dist.barrier()


def test_selfcheck_logic_two_ranks():
    spawn_ranks(_selfcheck_worker, 2, "gloo")


def _selfcheck_recovery_worker(rank, world_size):
    """A check that ends in a device-side timeout on ONE rank: every rank drops its symmetric memory,
    and the checks after it run on fresh allocations."""
    import torch.distributed as dist

    from symm_mem_recipes_b200 import selfcheck
    from symm_mem_recipes_b200.errors import SymmMemTimeout
    from symm_mem_recipes_b200.parallel import symm_mem

    seen = []

    def healthy():
        t = symm_mem.empty(64, dtype=torch.float32, device="cpu")
        hdl = symm_mem.rendezvous(t)
        t.fill_(float(rank + 1))
        hdl.barrier()
        total = sum(float(hdl.get_buffer(r, (64,), torch.float32)[0]) for r in range(world_size))
        hdl.barrier()
        seen.append(symm_mem.memory_summary()["count"])
        return total == sum(range(1, world_size + 1)), ""

    def times_out_on_rank_1():
        if rank == 1:
            raise SymmMemTimeout(3, rank, 0, 0, 1, 0)
        return True, ""

    checks = [("a", "healthy", False, healthy), ("a", "timeout on one rank", True, times_out_on_rank_1),
              ("a", "healthy again", False, healthy), ("a", "and again", False, healthy)]
    results, recoveries, stopped = selfcheck.run_checks(checks, rank, torch.device("cpu"))
    assert [r["ok"] for r in results] == [True, False, True, True], results
    assert recoveries == 1 and not stopped
    assert seen == [1, 1, 2]            # the allocation of the first check was dropped by the recovery
    dist.barrier()


def test_selfcheck_recovers_from_a_timeout_on_one_rank():
    spawn_ranks(_selfcheck_recovery_worker, 2, "gloo")

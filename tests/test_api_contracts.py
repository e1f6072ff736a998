"""Argument checking of the public ops: a wrong call must raise SymmMemError on
the host, before anything is launched.  Runs without a GPU."""
import pytest
import torch

import symm_mem_recipes_b200 as smr
from symm_mem_recipes_b200 import ops
from symm_mem_recipes_b200.errors import SymmMemError
from symm_mem_recipes_b200.ops.ag_matmul import AgMatmulConfig, _epilogue_code, choose_block_n


def _bf16(*shape):
    return torch.zeros(*shape, dtype=torch.bfloat16)


def test_gemm_ops_refuse_host_tensors_and_wrong_dtypes():
    with pytest.raises(SymmMemError, match="CUDA"):
        smr.matmul(_bf16(128, 64), _bf16(256, 64))
    with pytest.raises(SymmMemError, match="CUDA"):
        smr.all_gather_matmul(_bf16(128, 64), _bf16(256, 64))
    with pytest.raises(SymmMemError):
        smr.all_gather_matmul(torch.zeros(128, 64), torch.zeros(256, 64))           # fp32
    with pytest.raises(SymmMemError):
        smr.matmul(_bf16(2, 128, 64), _bf16(256, 64))                               # 3-D


def test_gemv_and_reduce_scatter_shape_checks():
    with pytest.raises(SymmMemError, match="x\\[B, K\\]"):
        smr.gemv_all_reduce(_bf16(4, 64), _bf16(32, 128))
    with pytest.raises(SymmMemError, match="between 1 and 16"):
        smr.gemv_all_reduce(_bf16(17, 64), _bf16(64, 128))
    with pytest.raises(SymmMemError, match="multiple of 8"):
        smr.gemv_all_reduce(_bf16(4, 64), _bf16(64, 100))
    with pytest.raises(SymmMemError, match="a\\[M, K\\]"):
        smr.matmul_reduce_scatter(_bf16(256, 64), _bf16(128, 32))


def test_layer_glue_refuses_host_tensors_and_odd_shapes():
    with pytest.raises(SymmMemError, match="CUDA"):
        ops.rms_norm(_bf16(4, 64), _bf16(64), 1e-5)
    with pytest.raises(SymmMemError, match="CUDA"):
        ops.rope_(_bf16(4, 256), 2, 64, 4, 10000.0)
    with pytest.raises(SymmMemError, match="CUDA"):
        ops.silu_mul(_bf16(4, 64))


def test_epilogue_and_tile_choices():
    cfg = AgMatmulConfig()
    assert _epilogue_code(None, torch.bfloat16, 1000, cfg) == 0
    assert _epilogue_code("swiglu", torch.bfloat16, 7168, cfg) == 1
    with pytest.raises(SymmMemError):
        _epilogue_code("gelu", torch.bfloat16, 7168, cfg)
    with pytest.raises(SymmMemError):
        _epilogue_code("swiglu", torch.bfloat16, 7168 + 128, cfg)                   # not whole 256-column tiles
    with pytest.raises(SymmMemError):
        _epilogue_code("swiglu", torch.float8_e4m3fn, 7168, cfg)
    with pytest.raises(SymmMemError):
        _epilogue_code("swiglu", torch.bfloat16, 7168, AgMatmulConfig(block_n=128))
    assert choose_block_n(4096, 100, 148) == 128 and choose_block_n(4096, 200, 148) == 224
    assert choose_block_n(4096, 3584, 148) == 256


def test_barrier_test_kinds_are_checked():
    class FakeHandle:
        kind = "cuda"
        has_multicast = False
        native = None

    with pytest.raises(SymmMemError, match="kind must be"):
        smr.barrier_test(FakeHandle(), kind="ring")
    with pytest.raises(SymmMemError, match="multicast"):
        smr.barrier_test(FakeHandle(), kind="nvls")


def test_matmul_all_reduce_shape_checks():
    with pytest.raises(SymmMemError, match="a\\[M, K\\]"):
        smr.matmul_all_reduce(_bf16(256, 64), _bf16(128, 32))


def test_info_runs_without_a_gpu():
    from symm_mem_recipes_b200 import info

    d = info.collect()
    assert "torch" in d and "gpus" in d and d["limits"]["max_world_size"] >= 8
    if not torch.cuda.is_available():
        assert d["gpus"] == [] and "CPU backend" in d["note"]


def test_timeout_messages_name_the_place():
    """Every `Where` code of the native status record has a description on the Python side."""
    import pathlib
    import re

    from symm_mem_recipes_b200 import errors

    header = (pathlib.Path(errors.__file__).parent / "csrc" / "device" / "status.h").read_text()
    body = header[header.index("enum Where"):]
    body = body[:body.index("};")]
    codes = {int(v) for v in re.findall(r"kWhere\w+\s*=\s*(\d+)", body)}
    assert codes and codes == set(errors._WHERE), (sorted(codes), sorted(errors._WHERE))
    e = errors.SymmMemTimeout(3, 1, 5, 0, 24, 7)
    assert "a gathered block never arrived" in str(e) and "rank=1" in str(e) and e.where == 24

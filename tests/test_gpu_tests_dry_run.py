"""The GPU tests' own code on the CPU.  The workers of the `gpu` tests (the
functions each rank runs) are executed here in gloo ranks with every CUDA
device mapped to the CPU and the kernels replaced by host stand-ins.  Their
numerics assertions then hold by construction; what is exercised is the test
code itself (shapes, references, argument lists), so that a typo in a test is
found here and not on its first GPU run."""
import importlib

import pytest
import torch

from symm_mem_recipes_b200.utils.testing import spawn_ranks

FACTORIES = ("randn", "zeros", "empty", "full", "ones", "arange", "tensor", "rand", "randint")


def _is_cuda(d) -> bool:
    return (isinstance(d, torch.device) and d.type == "cuda") or (isinstance(d, str) and d.startswith("cuda"))


def _map_cuda_to_cpu():
    """In this process, from here on: `device="cuda"` means the CPU."""
    for name in FACTORIES:
        real = getattr(torch, name)

        def factory(*a, _real=real, **k):
            if _is_cuda(k.get("device")):
                k.pop("device")
            return _real(*a, **k)

        setattr(torch, name, factory)
    real_to = torch.Tensor.to

    def to(self, *a, **k):
        a = tuple(x for x in a if not _is_cuda(x))
        if _is_cuda(k.get("device")):
            k.pop("device")
        return real_to(self, *a, **k) if (a or k) else self

    torch.Tensor.to = to
    torch.Tensor.cuda = lambda self, *a, **k: self
    torch.cuda.set_device = lambda d: None
    torch.cuda.synchronize = lambda d=None: None
    torch.cuda.device_count = lambda: 8
    from symm_mem_recipes_b200.parallel import symm_mem
    real_empty = symm_mem.empty

    def empty(*size, dtype=torch.float32, device=None):
        return real_empty(*size, dtype=dtype, device="cpu")

    symm_mem.empty = empty
    ag_mod = importlib.import_module("symm_mem_recipes_b200.ops.ag_matmul")
    real_gather_buffer = ag_mod.gather_buffer
    ag_mod.gather_buffer = lambda M, K, device, *a, **k: real_gather_buffer(M, K, torch.device("cpu"), *a, **k)
    import symm_mem_recipes_b200.utils.testing as testing
    real_guarded = testing.guarded_empty
    testing.guarded_empty = lambda shape, dtype, device, *a, **k: real_guarded(shape, dtype, "cpu", *a, **k)


def _eager_decode_graph():
    from symm_mem_recipes_b200.models import llama_tp_layer

    class EagerDecodeGraph:                            # same interface; replays by running the static step
        def __init__(self, layers, batch, max_seq, fused=True, warmup=2, caches=None):
            self.layers, self.fused, self.max_seq = list(layers), fused, max_seq
            cfg = self.layers[0].cfg
            self.pos = torch.zeros(1, dtype=torch.int32)
            self.caches = caches if caches is not None else [
                (torch.zeros(batch, max_seq, lyr.hkv, cfg.head_dim, dtype=torch.bfloat16),
                 torch.zeros(batch, max_seq, lyr.hkv, cfg.head_dim, dtype=torch.bfloat16)) for lyr in self.layers]

        def step(self, x, pos):
            from symm_mem_recipes_b200.models.llama_tp_layer import decode_static_through
            self.pos.fill_(pos)
            return decode_static_through(self.layers, self.caches, x, self.pos, fused=self.fused)

    llama_tp_layer.DecodeGraph = EagerDecodeGraph


def _dry(rank, world_size, module, fn_name, args, by_name):
    import test_fused_ops_flow_cpu as flow

    _map_cuda_to_cpu()
    flow._install_all_stand_ins()
    _eager_decode_graph()
    import symm_mem_recipes_b200 as smr
    smr.barrier_test = lambda hdl, num_blocks=32, **k: hdl.barrier()     # the kernel form exists on the GPU only
    mod = importlib.import_module(module)
    for dep in ("guarded_empty",):                     # names the test modules imported before the mapping
        if hasattr(mod, dep):
            import symm_mem_recipes_b200.utils.testing as testing
            setattr(mod, dep, getattr(testing, dep))
    fn = getattr(mod, fn_name)
    if by_name:                                        # a test function: keyword arguments, no rank
        result = fn(**args)
        assert not isinstance(result, int) or result == 0, f"{fn_name} returned {result}"   # a program's exit code
    else:
        fn(rank, world_size, *args)


WORKERS = [
    # module, worker, world sizes, arguments
    ("test_gpu_gemv", "_gemv_worker", (1, 2), (4, 256, 512, "tc_tagged")),
    ("test_gpu_gemv", "_gemv_nk_worker", (1, 2), (3, 256, 512, "tc_tagged")),
    ("test_gpu_matmul_fp8", "_mm_worker", (1,), (256, 512, 256, 256, 0, True)),
    ("test_gpu_matmul_fp8", "_agmm_worker", (2,), (128, 256, 256)),
    ("test_gpu_matmul_rs", "_ar_worker", (2,), (256, 256, 128)),
    ("test_gpu_llama_layer", "_layer_worker", (1, 2), ()),
    ("test_gpu_llama_layer", "_layer_tp_worker", (2,), (True, True)),
    ("test_gpu_llama_layer", "_decode_graph_worker", (1, 2), (True,)),
    ("test_gpu_llama_layer", "_stack_worker", (1, 2), ()),
    ("test_gpu_symm_mem", "_signals_gpu_worker", (2,), ()),
    ("test_gpu_symm_mem", "_compat_gpu_worker", (2,), ()),
    ("test_gpu_matmul", "_agmm_worker", (2,), (128, 256, 256, "plain")),
    ("test_gpu_matmul", "_agmm_worker", (2,), (128, 256, 256, "internal")),
    # the default forms of the multi-GPU tests
    ("test_gpu_matmul", "_agmm_worker", (2,), (128, 256, 256, "push_plain")),
    ("test_gpu_gemv", "_gemv_worker", (2,), (4, 256, 512, "tc")),
    ("test_gpu_matmul_rs", "_rs_worker", (2,), (256, 256, 128)),
]


@pytest.mark.parametrize("module,worker,worlds,args", WORKERS,
                         ids=[f"{m}.{w}{i}" for i, (m, w, _, _) in enumerate(WORKERS)])
def test_gpu_test_worker_runs_on_the_cpu(module, worker, worlds, args):
    mod = importlib.import_module(module)
    assert hasattr(mod, worker), f"{module} has no {worker}"
    for ws in worlds:
        spawn_ranks(_dry, ws, "gloo", (module, worker, args, False), timeout_s=240.0)


FUNCTIONS = [
    ("test_gpu_layer_glue", "test_rms_norm", {"rows": 37, "H": 512}),
    ("test_gpu_layer_glue", "test_rope", {"batch": 2, "seq": 24, "hq": 4, "hkv": 1, "D": 64, "pos0": 5}),
    ("test_gpu_layer_glue", "test_silu_mul", {"rows": 19, "F": 48}),
    ("test_gpu_layer_glue", "test_decode_attention", {"B": 3, "hq": 4, "hkv": 2, "D": 64, "s_max": 40,
                                                      "positions": (0, 7, 39)}),
    ("test_gpu_matmul", "test_matmul_small", {"block_n": 224, "shape": (200, 328, 96)}),
    ("test_gpu_layer_glue", "test_layer_with_fused_glue_matches_fp32", {}),
    ("test_gpu_layer_glue", "test_layer_with_fused_swiglu_matches_fp32", {}),
    ("test_gpu_layer_glue", "test_matmul_with_swiglu_epilogue", {"M": 200, "F": 384, "K": 96}),
    ("__graft_entry__", "smoke", {}),                  # the smoke check that runs on a GPU before the benchmark
    ("symm_mem_recipes_b200.selfcheck", "main", {"argv": []}),     # the one-GPU form of the self-check
    # the single-GPU tests that run at every GPU test pass
    ("test_gpu_symm_mem", "test_world_of_one_all_paths", {}),
    ("test_gpu_gemv", "test_gemv_world_of_one", {"B": 3, "K": 1000, "N": 328, "algo": "tc"}),
    ("test_gpu_gemv", "test_gemv_world_of_one", {"B": 8, "K": 256, "N": 64, "algo": "simt"}),
    ("test_gpu_matmul_rs", "test_matmul_reduce_scatter_world_of_one", {}),
    ("test_gpu_llama_layer", "test_layer_world_of_one", {}),
    ("test_gpu_matmul", "test_matmul_split_k_tail", {"shape": (768, 768, 1024), "num_sms": 8}),
]


@pytest.mark.parametrize("module,name,kwargs", FUNCTIONS,
                         ids=[f"{m}.{n}{i}" for i, (m, n, _) in enumerate(FUNCTIONS)])
def test_gpu_test_function_runs_on_the_cpu(module, name, kwargs):
    spawn_ranks(_dry, 1, "gloo", (module, name, kwargs, True), timeout_s=240.0)

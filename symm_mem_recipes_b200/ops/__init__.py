from .all_reduce import (all_reduce, choose_algo, low_latency_all_reduce,  # noqa: F401
                         multimem_all_reduce_, one_shot_all_reduce, two_shot_all_reduce_)
from .barrier import barrier_test, wait_flag  # noqa: F401
from .ag_matmul import (AgMatmulConfig, all_gather_matmul, interleave_gate_up, matmul,  # noqa: F401
                        reference_all_gather_matmul)
from .gemv_all_reduce import gemv, gemv_all_reduce, reference_gemv_all_reduce  # noqa: F401
from .matmul_reduce_scatter import (matmul_all_reduce, matmul_reduce_scatter,  # noqa: F401
                                    reference_matmul_all_reduce, reference_matmul_reduce_scatter)
from .layer_glue import decode_attention_, rms_norm, rope_, silu_mul  # noqa: F401

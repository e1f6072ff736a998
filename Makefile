# Common entry points.  Everything builds in tree; no GPU is needed for `build` and `test`.
PY ?= python
NPROC ?= 8
TORCHRUN = $(PY) -m torch.distributed.run --nnodes 1 --nproc-per-node $(NPROC) --master-addr 127.0.0.1

.PHONY: build test test-gpu selfcheck bench bench-suite bench-detail report expect clean

build:            ## nvcc -gencode arch=compute_100a,code=sm_100a for every kernel, link the extension
	$(PY) -m symm_mem_recipes_b200._build

test: build       ## oracles, host backend, gloo ranks, schedules, flow tests
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build   ## on a B200 box; multi-GPU cases skip when GPUs are missing
	$(PY) -m pytest tests -q -m gpu

selfcheck: build  ## every op once on small shapes in one start-up, NPROC GPUs (ARGS="--only gemv,glue" narrows it)
	if [ "$(NPROC)" = "1" ]; then $(PY) -m symm_mem_recipes_b200.selfcheck $(ARGS); \
	else $(TORCHRUN) -m symm_mem_recipes_b200.selfcheck $(ARGS); fi

bench: build      ## headline: all_gather_matmul at the Llama-3-70B TP shape, NPROC GPUs
	if [ "$(NPROC)" = "1" ]; then $(PY) bench.py --gpus 1; else $(TORCHRUN) bench.py --gpus $(NPROC); fi

bench-suite: build   ## every benchmark, JSON lines under out/
	mkdir -p out && $(TORCHRUN) -m symm_mem_recipes_b200.bench.suite --out-dir out --with-reference-triton

bench-detail: build  ## layer, GEMV and the upstream table with every opt-in kernel variant as guarded sections
	mkdir -p out && $(TORCHRUN) -m symm_mem_recipes_b200.bench.suite --out-dir out --layer-detail \
		--only layer,gemv,upstream_table

expect:           ## what the roofline allows for the 70B layer at NPROC ranks
	$(PY) -m symm_mem_recipes_b200.bench.expect layer_prefill --ws $(NPROC) --peaks MEASURED_PEAKS.json
	$(PY) -m symm_mem_recipes_b200.bench.expect layer_decode --ws $(NPROC) --peaks MEASURED_PEAKS.json

report:           ## Markdown tables with roofline fractions from out/*.jsonl
	$(PY) -m symm_mem_recipes_b200.bench.report out/*.jsonl --peaks MEASURED_PEAKS.json

clean:
	rm -rf build symm_mem_recipes_b200/_C*.so

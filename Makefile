# Common entry points.  Everything builds in tree; no GPU is needed for `build` and `test`.
PY ?= python
NPROC ?= 8
TORCHRUN = $(PY) -m torch.distributed.run --nnodes 1 --nproc-per-node $(NPROC) --master-addr 127.0.0.1

.PHONY: build test test-gpu test-first-run bench bench-suite report clean

build:            ## nvcc -gencode arch=compute_100a,code=sm_100a for every kernel, link the extension
	$(PY) -m symm_mem_recipes_b200._build

test: build       ## oracles, host backend, gloo ranks, schedules, flow tests
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build   ## on a B200 box; multi-GPU cases skip when GPUs are missing
	$(PY) -m pytest tests -q -m gpu

test-first-run: build   ## also the variants whose first run on hardware is pending
	SMR_TEST_FIRST_RUN=1 $(PY) -m pytest tests -q -m gpu

bench: build      ## headline: all_gather_matmul at the Llama-3-70B TP shape, NPROC GPUs
	if [ "$(NPROC)" = "1" ]; then $(PY) bench.py --gpus 1; else $(TORCHRUN) bench.py --gpus $(NPROC); fi

bench-suite: build   ## every benchmark, JSON lines under out/
	mkdir -p out && $(TORCHRUN) -m symm_mem_recipes_b200.bench.suite --out-dir out --with-reference-triton

report:           ## Markdown tables with roofline fractions from out/*.jsonl
	$(PY) -m symm_mem_recipes_b200.bench.report out/*.jsonl --peaks MEASURED_PEAKS.json

clean:
	rm -rf build symm_mem_recipes_b200/_C*.so

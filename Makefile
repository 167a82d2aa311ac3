# Developer entry points. Everything runs from the repository root with the interpreter on PATH.
PYTHON ?= python

.PHONY: build test test-gpu bench bench-reference microbench style clean

build:            ## cross-compile csrc/ for sm_100a into csrc/_build/ (works without a GPU)
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

test:             ## CPU suite: single process and gloo multi-rank
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu: build   ## kernels and models on a B200 (multi-GPU checks need >= 2 devices)
	$(PYTHON) -m pytest tests -q -m gpu

bench: build      ## headline benchmark on one GPU (dense 8B + the MoE record), one JSON line
	$(PYTHON) bench.py --gpus 1 --steps 3 --warmup 3

bench-reference:  ## the unmodified reference from baseline/_ref on the same metric
	$(PYTHON) bench.py --impl reference --gpus 1 --steps 3 --warmup 3

microbench: build ## kernel micro-benchmarks
	$(PYTHON) -m lm_engine.ops.microbench gemm
	$(PYTHON) -m lm_engine.ops.microbench mxfp8
	$(PYTHON) -m lm_engine.ops.microbench attention

style:            ## the pre-commit hooks over the whole tree
	pre-commit run --all-files

clean:
	rm -rf csrc/_build

# Convenience targets; every recipe is one command that can also be run by hand.
PY ?= python

.PHONY: build test test-gpu bench bench-library kernels regression examples notebooks docs-check sanitize clean

build:            ## compile the CUDA library (nvcc, sm_100a) and the host library (g++) in-tree
	$(PY) __graft_entry__.py

test: build       ## CPU suite (multi-process paths on gloo)
	$(PY) -m pytest tests -q -m "not gpu"

test-gpu: build   ## on a B200
	$(PY) -m pytest tests -q -m gpu

bench:            ## flagship training step on one GPU, one JSON line
	$(PY) bench.py --gpus 1 --steps 6 --warmup 3

bench-library:    ## the same step in PyTorch library ops (comparator)
	$(PY) bench.py --impl library --gpus 1 --steps 6 --warmup 3

kernels:          ## per-kernel roofline fractions
	$(PY) -m sneppx_alg_b200.benchmarks.kernels all --out kernels.json

regression: kernels  ## fail when a kernel fell below its stored floor
	$(PY) -m sneppx_alg_b200.benchmarks.regression kernels.json

examples:         ## run every example
	for f in examples/ex_*.py; do $(PY) $$f || exit 1; done

notebooks:        ## regenerate examples/notebooks from the scripts
	$(PY) examples/to_notebook.py --all

docs-check:       ## execute the runnable blocks of docs/ and check links
	$(PY) -m pytest tests/test_docs_cpu.py tests/test_examples_cpu.py -q

sanitize:         ## host library under AddressSanitizer + UBSan; prints the path to give to SX_HOST_LIB
	$(PY) -c "from sneppx_alg_b200 import _build; print(_build.build_host_sanitized(kind='address'))"

clean:
	rm -rf sneppx_alg_b200/lib/obj kernels.json

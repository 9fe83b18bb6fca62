# Build the sm_100a extension in-tree and run the test tiers.
PYTHON ?= python

.PHONY: build test test-gpu test-multi-gpu bench

build:
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

test:
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu: build
	$(PYTHON) -m pytest tests -x -q -m gpu

test-multi-gpu: build
	$(PYTHON) -m pytest tests/test_gpu_multi.py -x -q

bench: build
	$(PYTHON) bench.py --gpus 1

# Common developer commands.

build:
	python -m makani_b200.csrc.build

install: build
	pip install -e .

test:
	python -m pytest tests -q -m "not gpu"

test-gpu:
	python -m pytest tests -q -m gpu

bench:
	python bench.py --gpus 1 --steps 10 --warmup 3

kernels:
	python -m makani_b200.utils.kernel_bench

quickstart:
	python examples/quickstart.py

.PHONY: build install test test-gpu bench kernels quickstart

.PHONY: all build clean test test-gpu sanitize check python-smoke release-check bench

PYTHON ?= python

# Default target: build everything in-tree (C++ core, sm_100a kernels, torch glue, tools, circuit simulator)
all: build

build:
	$(PYTHON) -m nangila._build

# Remove what the build writes; sources are never touched
clean:
	rm -rf build
	rm -f nangila/_C*.so nangila/_cuda*.so nangila/libnangila_kernels.so
	rm -f nangila_spice/_native*.so nangila_spice/bin/nangila-node
	rm -f nangila/cli/nangila-dump nangila/cli/nangila-profile
	rm -rf tests/__pycache__ examples/__pycache__ bench/__pycache__

# CPU tier: core, gloo DDP, fault injection, resume, tools, models, circuit simulator
test:
	$(PYTHON) -m pytest tests -q -m "not gpu"

# B200 tier: kernel numerics against fp32 PyTorch, multi-GPU workers
test-gpu:
	$(PYTHON) -m pytest tests -q -m gpu

# Host code under AddressSanitizer + UndefinedBehaviorSanitizer against hostile input (part of `make test` as well)
sanitize:
	$(PYTHON) -m pytest tests/test_sanitizers_cpu.py -q

# Does everything compile (nvcc cross-compiles without a GPU) and import
check:
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

# The quick import + round-trip check a fresh checkout should pass
python-smoke: build
	$(PYTHON) -m pytest tests/test_core.py tests/test_cli_and_cabi.py -q

# The documented local release validation: manifest against the tree, then the CPU tier
release-check:
	$(PYTHON) -m nangila.cli.release_check
	$(MAKE) test

bench:
	$(PYTHON) bench.py --gpus 1 --steps 20 --warmup 5

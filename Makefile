.PHONY: help build build-debug rebuild ptxas test-cpu test-gpu sanitize bench bench-reference example lint clean

PYTHON ?= python
NGPU ?= 1
TORCHRUN = $(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NGPU) --master-addr 127.0.0.1

help:  ## Show this help
	@grep -E '^[a-zA-Z_-]+:.*?## .*$$' $(MAKEFILE_LIST) | sort | \
		awk 'BEGIN {FS = ":.*?## "}; {printf "%-16s %s\n", $$1, $$2}'

build:  ## Compile csrc/ for sm_100a into tileccl_b200/lib/libtileccl_b200.so (no GPU needed)
	$(PYTHON) -m tileccl_b200._build

build-debug:  ## The same sources with recorded bounds checks (-DTILECCL_DEBUG_CHECKS; TILECCL_DEBUG=1 loads it)
	$(PYTHON) -m tileccl_b200._build --debug

rebuild:  ## Recompile everything (release and debug libraries)
	$(PYTHON) -m tileccl_b200._build --all --force

sanitize:  ## CPU emulation of the signalling protocol under ThreadSanitizer and ASan/UBSan
	$(PYTHON) -m pytest tests/test_emulator_sanitizers.py -q

ptxas:  ## Print registers / spills / shared memory of every kernel
	$(PYTHON) -m tileccl_b200._build --ptxas-v

test-cpu: build build-debug  ## Tests that need no GPU (planning, emulator, bootstrap, build checks)
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu: build build-debug  ## Tests that need a B200
	$(PYTHON) -m pytest tests -x -q -m gpu

bench: build  ## Headline benchmark on NGPU GPUs (make bench NGPU=8)
ifeq ($(NGPU),1)
	$(PYTHON) bench.py --gpus 1
else
	$(TORCHRUN) bench.py --gpus $(NGPU)
endif

bench-reference:  ## The same benchmark through the unmodified reference in baseline/_ref
ifeq ($(NGPU),1)
	$(PYTHON) bench.py --impl reference --gpus 1
else
	$(TORCHRUN) bench.py --impl reference --gpus $(NGPU)
endif

example: build  ## User kernel built on the device primitives, emulated ranks on one GPU
	$(PYTHON) examples/custom_kernel.py

lint:  ## ruff, when installed
	ruff check tileccl_b200 tileccl tileccl_v2 tests examples benchmarks bench.py

clean:  ## Remove build artefacts
	rm -rf build/ dist/ *.egg-info .pytest_cache .ruff_cache tileccl_b200/lib/libtileccl_b200.so tileccl_b200/lib/libtileccl_b200_debug.so
	find . -type d -name __pycache__ -prune -exec rm -rf {} + 2>/dev/null || true

# Convenience targets; every command also works on its own.
PYTHON ?= python
NP ?= 4

.PHONY: build test test-gpu examples bench bench-reference tsan-build tsan clean

build:            ## compile the C++/CUDA extension for sm_100a into bluefog_b200/
	$(PYTHON) setup.py build_ext --inplace

test:             ## CPU ranks over TCP + shared memory (no GPU needed)
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu:         ## kernels, models and multi-GPU ops (skips what the box has too few GPUs for)
	$(PYTHON) -m pytest tests -q -m gpu

examples:         ## the example scripts end to end on CPU ranks
	$(PYTHON) -m pytest tests/test_examples_cpu.py -q

bench:            ## flagship benchmark on one GPU; for N GPUs: torchrun --nproc-per-node N bench.py --gpus N
	$(PYTHON) bench.py --gpus 1

bench-reference:  ## the reference arm (prints why it is unavailable when the reference cannot be built)
	$(PYTHON) bench.py --impl reference --gpus 1

tsan-build:       ## ThreadSanitizer build of the host runtime, beside the regular library (needs a g++ with libtsan)
	CC=/usr/bin/gcc CXX=/usr/bin/g++ BLUEFOG_B200_TSAN=1 $(PYTHON) setup.py build_ext --build-lib build/tsan --build-temp build/tsan_tmp

tsan: tsan-build  ## multi-process CPU cases against that build; fails on any report tests/tsan.supp does not cover
	$(PYTHON) tests/tsan_check.py --ranks $(NP)

clean:
	rm -rf build bluefog_b200/_C*.so

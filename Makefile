# Builds the two native libraries in-tree and runs the test tiers.
#   make            both libraries
#   make kernels    sm_100a kernel library (nvcc cross-compiles without a GPU)
#   make runtime    host runtime: engine, storage, file formats, C interface
#   make test       CPU test tier        make test-gpu   GPU test tier (needs a B200)
#   make capi       the plain-C program of the C interface
PYTHON ?= python
NVCC   ?= /usr/local/cuda/bin/nvcc

.PHONY: all kernels runtime test test-gpu capi docs clean

all: kernels runtime

kernels:
	NVCC=$(NVCC) $(PYTHON) -m mxnet_b200.ops.cuda.build

runtime:
	$(PYTHON) -c "from mxnet_b200.csrc import runtime; print(runtime.build_runtime(force=True))"

test: all
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu: all
	$(PYTHON) -m pytest tests -q -m gpu

capi: runtime
	gcc -std=c11 -O1 -Wall -I mxnet_b200/include cpp-package/tests/c_api_test.c -o c_api_test \
	    -L mxnet_b200/csrc -lmxb200_rt -lm -Wl,-rpath,$(CURDIR)/mxnet_b200/csrc

docs:
	$(PYTHON) -c "from mxnet_b200 import env; open('docs/env_var.md', 'w').write(env.markdown())"

clean:
	rm -rf mxnet_b200/ops/cuda/build
	rm -f mxnet_b200/ops/cuda/libmxb200_kernels.so mxnet_b200/csrc/libmxb200_rt.so c_api_test

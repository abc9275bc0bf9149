# Developer entry points.  The kernels are built in-tree; nothing is installed outside the checkout.
PYTHON ?= python

.PHONY: build test test-gpu sanitize bench clean

build:            ## nvcc (sm_100a) + g++: libb200ops.so, libb200host.so, devquery
	$(PYTHON) -m ollama_b200.kernels.build

test: build       ## everything that needs no GPU
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu: build   ## on a B200
	$(PYTHON) -m pytest tests -x -q -m gpu

sanitize:         ## host C++ under AddressSanitizer + UndefinedBehaviorSanitizer
	$(PYTHON) -m ollama_b200.native.sanitize

bench: build
	$(PYTHON) bench.py

clean:
	rm -rf ollama_b200/kernels/build ollama_b200/kernels/libb200ops.so ollama_b200/native/libb200host.so ollama_b200/native/devquery

# Convenience targets; everything they do is a python entry point (the build itself is skygdr_b200/build.py).
# The reference builds with two Makefiles (src/Makefile, llm_problem_analysis/Makefile); users of those find the same verbs here.
PYTHON ?= python

.PHONY: all ctl bin cuda test test-gpu bench smoke clean

all:            ## control plane (g++), host programs, sm_100a kernels (nvcc); no GPU needed
	$(PYTHON) -m skygdr_b200.build all

ctl:
	$(PYTHON) -m skygdr_b200.build ctl

bin:
	$(PYTHON) -m skygdr_b200.build bin

cuda:
	$(PYTHON) -m skygdr_b200.build cuda

test:           ## CPU tests
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu:       ## needs a B200
	$(PYTHON) -m pytest tests -q -m gpu

bench:          ## Qwen3-8B decode tokens/s on one GPU
	$(PYTHON) bench.py --gpus 1

smoke:
	$(PYTHON) __graft_entry__.py smoke

clean:
	rm -rf skygdr_b200/build skygdr_b200/bin skygdr_b200/_C*.so skygdr_b200/_ctl*.so

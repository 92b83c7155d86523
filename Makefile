# Convenience targets (the reference's Makefile has build / clean / test-cpp).
PYTHON ?= python

build:
	$(PYTHON) -c "import __graft_entry__ as g; g.build()"

clean:
	rm -rf build/titb200
	rm -f tinyinfinitrain_b200/_C.so tinyinfinitrain_b200/libtitb200_kernels.so

cpp:
	$(PYTHON) -m tinyinfinitrain_b200._build --cpp

test-cpu: build
	$(PYTHON) -m pytest tests -q -m "not gpu"

test-gpu: build
	$(PYTHON) -m pytest tests -q -m gpu

bench: build
	$(PYTHON) bench.py --gpus 1 --steps 20 --warmup 5

.PHONY: build cpp clean test-cpu test-gpu bench

# Convenience targets (the reference's Makefile:19-102 offers install/build/node/orchestui/cluster-up/bench/test).
PY ?= python
NODES ?= 3
BASE_PORT ?= 40000

.PHONY: build test test-gpu sanitize node orchestui orchestrator cluster-up bench bench-nccl bench-kernels clean

build:            ## CUDA kernels (sm_100a), the C++ core extension and the native executables
	$(PY) -c "import __graft_entry__ as g; g.build()"

test: build       ## CPU test-suite
	$(PY) -m pytest tests -x -q -m "not gpu"

test-gpu: build   ## needs a B200
	$(PY) -m pytest tests -x -q -m gpu

sanitize:         ## sessions through ASan+UBSan and TSan builds of the native executables
	$(PY) -m pytest tests/test_sanitizers_cpu.py -x -q

node: build       ## one listening node: make node PORT=40000 [GPU=0]
	PORT=$(PORT) ./bin/ono-node $(if $(GPU),--gpu $(GPU),--device cpu)

orchestui: build
	./bin/orchestui

orchestrator: build   ## make orchestrator MODEL=model.json TRAINING=training.json
	./bin/ono-orchestrator $(MODEL) $(TRAINING)

cluster-up: build ## NODES listening nodes on BASE_PORT.. (foreground; ctrl-c stops them)
	$(PY) -m oxidized_neural_orchestra_b200.runtime.launch --nodes $(NODES) --base-port $(BASE_PORT)

bench:
	$(PY) bench.py

bench-nccl:
	$(PY) bench.py --impl nccl

bench-kernels:
	$(PY) bench/kernels.py gemm && $(PY) bench/kernels.py sync

clean:
	rm -rf build bin/ono-node bin/ono-orchestrator bin/orchestui

# Convenience targets (the reference's Makefile:19-102 offers install/build/node/orchestui/cluster-up/bench/test).
PY ?= python
NODES ?= 3
BASE_PORT ?= 40000

.PHONY: build test test-gpu sanitize node orchestui orchestrator cluster-up cluster-down compose-up compose-down bench bench-nccl bench-kernels bench-suites bench-plots lint check clean

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
	$(PY) -m oxidized_neural_orchestra_b200.runtime.launch --nodes $(NODES) --base-port $(BASE_PORT) --pid-file .cluster.pid

cluster-down:     ## stop the nodes of a running `make cluster-up` (from another shell)
	@if [ -f .cluster.pid ]; then kill `cat .cluster.pid` && rm -f .cluster.pid; else echo "no .cluster.pid: nothing to stop"; fi

compose-up:       ## NODES node containers, one GPU each: make compose-up NODES=8 [RATE=10mbit]
	$(PY) docker/compose_up.py --nodes $(NODES) --base-port $(BASE_PORT) $(if $(RATE),--rate $(RATE),)

compose-down:
	$(PY) docker/compose_up.py --down

bench:
	$(PY) bench.py

bench-suites:     ## the reference's benchmark suites (strategies; SUITE=scalability|offline) -> bench/results/
	$(PY) bench/suites.py --suite $(or $(SUITE),strategies)

bench-plots:      ## SVG charts + plots.md from bench/results/history.jsonl
	$(PY) bench/plots.py

lint:             ## syntax check of every Python file, warnings-as-errors compile of the C++ core headers
	$(PY) -m compileall -q oxidized_neural_orchestra_b200 orchestra bench baseline examples docker tests bench.py __graft_entry__.py
	$(CXX) -std=c++17 -Wall -Wextra -Werror -Wno-unused-parameter -Wno-unused-function -fsyntax-only -I csrc csrc/core/configs.cpp csrc/core/codec.cpp

check: lint test  ## what CI runs

bench-nccl:
	$(PY) bench.py --impl nccl

bench-kernels:
	$(PY) bench/kernels.py gemm && $(PY) bench/kernels.py sync

clean:
	rm -rf build bin/ono-node bin/ono-orchestrator bin/orchestui

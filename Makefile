# usage: make help

.PHONY: help build test test-cpu test-gpu check docs bench
.DEFAULT_GOAL := help

help: ## this help
	@awk 'BEGIN {FS = ":.*##"} /^[0-9a-zA-Z_-]+:.*##/ { printf "  %-12s %s\n", $$1, $$2 }' $(MAKEFILE_LIST)

build: ## compile the CUDA extensions for sm_100a into csrc/build/ (no GPU needed)
	python -c "import __graft_entry__ as g; g.build()"

test: test-cpu test-gpu ## CPU tests, then GPU tests

test-cpu: ## tests that need no GPU (include 2-rank Gloo runs)
	python -m pytest tests -q -m "not gpu"

test-gpu: ## tests that need a B200
	python -m pytest tests -q -m gpu

check: ## source rules, licence headers, generated docs
	python ci/check_source_rules.py
	python ci/check_license.py
	python docs/gen_config_reference.py --check

docs: ## regenerate docs/config.md from the config classes
	python docs/gen_config_reference.py

bench: ## the headline benchmark on one GPU
	python bench.py --steps 5 --warmup 3

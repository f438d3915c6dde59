.PHONY: build test test-gpu bench lint docs serve

build:            ## compile every CUDA source for sm_100a (in-tree, no GPU needed)
	python -c "import __graft_entry__ as g; g.build()"

test:             ## CPU tests (multi-process ones use gloo on 127.0.0.1)
	python -m pytest tests -x -q -m "not gpu"

test-gpu:         ## needs a B200; the multi-GPU tests need two
	python -m pytest tests -x -q -m gpu

bench:            ## headline benchmark on one GPU
	python bench.py --gpus 1 --steps 20 --warmup 5

lint:
	ruff check language_model_saes_b200 tests bench.py

docs:
	mkdocs build

serve:            ## browse the embedded store under ./store
	MONGO_URI=file://$(PWD)/store uvicorn language_model_saes_b200.server.app:app --port 24577

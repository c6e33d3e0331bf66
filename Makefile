# Developer entry points.  Everything is built in-tree; nothing is downloaded.
PYTHON ?= python

.PHONY: build kernels router test test-gpu bench smoke clean

build: kernels router

kernels:          ## nvcc -gencode arch=compute_100a,code=sm_100a -> text-generation-inference_b200/ops/*.so
	$(PYTHON) -m tgi_b200.ops.build

router:           ## g++ -std=c++17 -> tgi-b200-router, tgi-b200-launcher, tgi-b200-benchmark
	$(PYTHON) -m tgi_b200.router.build

test:             ## CPU suite (multi-rank paths run on gloo)
	$(PYTHON) -m pytest tests -x -q -m "not gpu"

test-gpu:         ## needs a B200
	$(PYTHON) -m pytest tests -x -q -m gpu

smoke:
	$(PYTHON) -c "import __graft_entry__ as g; g.build(); g.smoke()"

bench:            ## headline decode benchmark on one GPU; `make bench GPUS=2` runs it tensor parallel
ifeq ($(or $(GPUS),1),1)
	$(PYTHON) bench.py
else
	$(PYTHON) -m torch.distributed.run --nnodes=1 --nproc-per-node $(GPUS) --master-addr 127.0.0.1 --master-port 29500 \
	    bench.py --gpus $(GPUS)
endif

clean:
	rm -f text-generation-inference_b200/ops/libtgi_b200_kernels.so
	rm -f text-generation-inference_b200/router/tgi-b200-router text-generation-inference_b200/router/tgi-b200-launcher \
	    text-generation-inference_b200/router/tgi-b200-benchmark

# One image for B200 (sm_100a): CUDA 12.9 toolchain, PyTorch, the in-tree kernel library and the C++ router.
#   docker build -t tgi-b200 .
#   docker run --gpus all --shm-size 1g -p 8080:80 -v $PWD/data:/data tgi-b200 --model-id /data/model --num-shard 8
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04 AS build
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv python3-dev g++ \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir torch numpy safetensors tokenizers transformers jinja2 protobuf grpcio pillow requests
WORKDIR /opt/tgi
COPY text-generation-inference_b200 text-generation-inference_b200
COPY tgi_b200 tgi_b200
ENV PYTHONPATH=/opt/tgi
# kernels: nvcc -gencode arch=compute_100a,code=sm_100a (no GPU needed to compile); router: g++ -std=c++17
RUN python -m tgi_b200.ops.build && python -m tgi_b200.router.build

FROM nvidia/cuda:12.9.0-runtime-ubuntu24.04
RUN apt-get update && apt-get install -y --no-install-recommends python3 libpython3.12 \
    && rm -rf /var/lib/apt/lists/*
COPY --from=build /opt/venv /opt/venv
COPY --from=build /opt/tgi /opt/tgi
COPY tgi-entrypoint.sh sagemaker-entrypoint.sh /usr/local/bin/
ENV PATH=/opt/venv/bin:/opt/tgi/text-generation-inference_b200/router:$PATH PYTHONPATH=/opt/tgi \
    HF_HOME=/data HF_HUB_OFFLINE=1 PORT=80
ENTRYPOINT ["tgi-entrypoint.sh"]

# Serving image: CUDA 12.9 toolchain to build the sm_100a kernels, then the same base to run them.
ARG CUDA=12.9.1
FROM nvidia/cuda:${CUDA}-devel-ubuntu24.04 AS build
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv g++ && rm -rf /var/lib/apt/lists/*
WORKDIR /src
COPY pyproject.toml setup.py README.md ./
COPY ollama_b200 ollama_b200
RUN python3 -m venv /opt/venv && /opt/venv/bin/pip install --no-cache-dir torch --index-url https://download.pytorch.org/whl/cu128 \
 && /opt/venv/bin/pip install --no-cache-dir .

FROM nvidia/cuda:${CUDA}-runtime-ubuntu24.04
RUN apt-get update && apt-get install -y --no-install-recommends python3 && rm -rf /var/lib/apt/lists/*
COPY --from=build /opt/venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH OLLAMA_HOST=0.0.0.0:11434 OLLAMA_MODELS=/models
VOLUME /models
EXPOSE 11434
ENTRYPOINT ["ollama-b200"]
CMD ["serve"]

# Build image for the framework and its sm_100a kernels (nvcc cross-compiles without a GPU).
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04
RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-dev ninja-build git && rm -rf /var/lib/apt/lists/*
WORKDIR /opt/lmsae
COPY . .
RUN pip install --break-system-packages torch --index-url https://download.pytorch.org/whl/cu128 && \
    pip install --break-system-packages -e ".[server]" && \
    python3 -c "import __graft_entry__ as g; g.build()"
ENV MONGO_URI=file:///data/store MONGO_DB=mechinterp
EXPOSE 24577
CMD ["uvicorn", "language_model_saes_b200.server.app:app", "--host", "0.0.0.0", "--port", "24577"]

# Build the llark_b200 C-ABI library (sm_100a only).
NVCC ?= /usr/local/cuda/bin/nvcc
ARCH := -gencode arch=compute_100a,code=sm_100a
NVFLAGS := $(ARCH) -std=c++17 -O3 -lineinfo -Xcompiler -fPIC -Xptxas -v
SRC := $(wildcard llark_b200/csrc/*.cu)
OBJ := $(patsubst llark_b200/csrc/%.cu,build/%.o,$(SRC))
LIB := llark_b200/libllark_b200.so

# the subset a native checkpoint of a layer-list decoder needs: GEMM core, decode linears, generation-path ops
SERVE_OBJ := build/gemm_tcgen05.o build/gemv.o build/seq_ops.o build/seq_mixers.o build/seq_swa_mma.o build/seq_delta.o \
             build/seq_latent.o build/seq_moe.o
LIB_SERVE := llark_b200/libllark_serve.so

all: $(LIB)
serve: $(LIB_SERVE)

build/%.o: llark_b200/csrc/%.cu llark_b200/csrc/common.cuh include/llark_b200.h
	@mkdir -p build
	$(NVCC) $(NVFLAGS) -c $< -o $@ 2> build/$*.ptxas.log || (cat build/$*.ptxas.log; exit 1)

# the ALiBi instantiation #includes the attention source: rebuild it when that changes
build/attention_tc_alibi.o: llark_b200/csrc/attention_tc.cu

$(LIB): $(OBJ)
	$(NVCC) $(ARCH) -shared -o $@ $(OBJ) -lnccl

$(LIB_SERVE): $(SERVE_OBJ)
	$(NVCC) $(ARCH) -shared -o $@ $(SERVE_OBJ)

clean:
	rm -rf build $(LIB) $(LIB_SERVE)
.PHONY: all serve clean

# Same targets as the reference's makefile (makefile:13-22): `make` builds the benchmark CLI a.out,
# `make share_lib` / `make lib` build libonebitmul.so / libonebitmul.a, `make lib_test` the link smoke
# test. Everything is compiled for sm_100a only; no CUTLASS is needed.
ROOT=.
PKG=$(ROOT)/onebitsparsemul_b200
CSRC=$(PKG)/csrc
NVCC=/usr/local/cuda/bin/nvcc
NVCC_FLAGS=-gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 --expt-relaxed-constexpr -I$(ROOT)/include
LIB_SRCS=$(CSRC)/api.cu $(CSRC)/pack.cu $(CSRC)/mask.cu $(CSRC)/relayout.cu $(CSRC)/gemm_simple.cu \
         $(CSRC)/gemm_decode.cu $(CSRC)/gemm_decode_sm100.cu $(CSRC)/gemm_prefill_sm100.cu $(CSRC)/gemm_prefill2_sm100.cu $(CSRC)/gemm_prefill3_sm100.cu $(CSRC)/gemm_prefill_splitk_sm100.cu $(CSRC)/noalloc.cu $(CSRC)/host_pipeline.cu

kernel: share_lib
	$(NVCC) $(NVCC_FLAGS) $(CSRC)/kernel_test.cu -o a.out -L$(PKG) -lonebitmul -Xlinker -rpath='$$ORIGIN/onebitsparsemul_b200'

share_lib:
	$(NVCC) $(NVCC_FLAGS) $(LIB_SRCS) -shared --compiler-options -fPIC -o $(PKG)/libonebitmul.so
	cp $(PKG)/libonebitmul.so libonebitmul.so

lib:
	$(NVCC) $(NVCC_FLAGS) $(LIB_SRCS) -lib --compiler-options -fPIC -o libonebitmul.a

lib_test: share_lib
	$(NVCC) $(NVCC_FLAGS) tests/libso_test.cu -o libso_test -L$(ROOT) -lonebitmul -Xlinker -rpath='$$ORIGIN'

torch_ext:
	python -c "from onebitsparsemul_b200 import build; print(build.build_torch_extension())"

clean:
	rm -f a.out libso_test libonebitmul.so libonebitmul.a $(PKG)/libonebitmul.so
	rm -rf $(PKG)/build

.PHONY: kernel share_lib lib lib_test torch_ext clean

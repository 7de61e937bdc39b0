# Builds the reference library twice from the sources where they lie (REF), with compile
# rules written here -- the reference's own CMake is not run:
#
#   _ref/tt_cpu/libtinytensor.a      the unmodified reference, CPU backend only.  Checker:
#                                    tinytensor::matmul, backward() and Generator behind C entry
#                                    points (_ref/libttref_full.so, from ref_full_driver.cpp).
#   _ref/tt_dropin/                  the reference WITH its CUDA backend (TT_CUDA, sm_100a), where
#                                    - backend/cuda/matmul.cu is left out and
#                                      tinytensor_b200/csrc/tt_runner_shim.cu defines its runner,
#                                    - backend/cuda/conv.cu keeps its pooling runners; its two
#                                      conv2d runners are compiled under other names and
#                                      csrc/tt_conv_shim.cu defines the real ones,
#                                    - backend/cuda/data_types.cu (DeviceMemory<T>) is compiled
#                                      with csrc/tt_alloc_shim.h force-included, which sends its
#                                      cudaMalloc / cudaFree to libttb.so's memory pool,
#                                    - autograd/unary_ops.cpp compiles its TensorToDevice under
#                                      another name and csrc/tt_to_device_shim.cpp defines it,
#                                    - backend/cuda/reduce.cu compiles its reduce_all_runner under
#                                      another name and csrc/tt_reduce_all_shim.cu defines it through
#                                      reduce_dim_runner (the reference's reduce_all_kernel reads past
#                                      its shared arrays, which faults on sm_100a; `allclose` in
#                                      every reference test runs it),
#                                    linked once into _ref/tt_dropin/libtinytensor_dropin.so
#                                    (default symbol visibility, so the small test executables
#                                    can share it), and the reference's own doctest executables
#                                    linked against it and libttb.so: _ref/tt_dropin/bin/test_*.
#
# Nothing of the reference is edited or copied: the substitutions are -D / -include flags on
# single translation units.  Outputs go only into _ref/ (git-ignored).
#
# Usage: make -f oracle/dropin.mk REF=<reference tree> [-j8] [cpu|dropin|all]
REF ?= $(TINYTENSOR_REFERENCE)
CXX ?= g++
NVCC ?= nvcc
PYTHON ?= python
HERE := $(dir $(abspath $(lastword $(MAKEFILE_LIST))))
ROOT := $(abspath $(HERE)..)
OUT := $(HERE)_ref
CSRC := $(ROOT)/tinytensor_b200/csrc
CUDA_HOME ?= /usr/local/cuda
TORCH_DIR := $(shell $(PYTHON) -c "import os, torch; print(os.path.dirname(torch.__file__))" 2>/dev/null)

ifeq ($(strip $(REF)),)
$(error set REF (or TINYTENSOR_REFERENCE) to the tinytensor source tree)
endif

GEN := $(OUT)/gen
INCLUDES := -I$(REF)/include -I$(REF)/tinytensor -isystem $(REF)/external/libnop/include -I$(GEN)
# The reference's release flags (CMakePresets.json: -O3 -DNDEBUG; CMakeLists.txt:11-15 hidden
# visibility, :71-74 -march): x86-64-v3 instead of native because the objects are built in one
# container and run on another host.
CXXFLAGS_BASE := -std=c++20 -O3 -DNDEBUG -march=x86-64-v3 -fPIC -DTINYTENSOR_STATIC_DEFINE -w $(INCLUDES)
CXXFLAGS := $(CXXFLAGS_BASE) -fvisibility=hidden -fvisibility-inlines-hidden
# CMakeLists.txt:52-62: --expt-relaxed-constexpr, separable compilation, TT_CUDA.
NVFLAGS := -gencode arch=compute_100a,code=sm_100a -std=c++20 --expt-relaxed-constexpr -rdc=true -O3 -DNDEBUG \
	-DTT_CUDA -DTINYTENSOR_STATIC_DEFINE -w -Xcompiler -fPIC,-march=x86-64-v3 $(INCLUDES)

# ---- source lists (relative to $(REF)/tinytensor) ---------------------------------------
CPP_ALL := $(patsubst $(REF)/tinytensor/%,%,$(shell find $(REF)/tinytensor -name '*.cpp' | sort))
CPP_CPU := $(filter-out tensor/backend/cuda/%,$(CPP_ALL))
# with TT_CUDA, random.cpp is compiled as CUDA (tinytensor/tensor/CMakeLists.txt:20)
CPP_DROPIN := $(filter-out tensor/random.cpp,$(CPP_ALL))
CU_ALL := $(patsubst $(REF)/tinytensor/%,%,$(shell find $(REF)/tinytensor -name '*.cu' | sort))
CU_DROPIN := $(filter-out tensor/backend/cuda/matmul.cu,$(CU_ALL))

flat = $(subst /,__,$(basename $(1)))
CPU_DIR := $(OUT)/tt_cpu
DI_DIR := $(OUT)/tt_dropin
LIBTTB := $(ROOT)/tinytensor_b200/libttb.so
DI_LIB := $(DI_DIR)/libtinytensor_dropin.so
CPU_OBJS := $(foreach s,$(CPP_CPU),$(CPU_DIR)/obj/$(call flat,$(s)).o)
DI_CPP_OBJS := $(foreach s,$(CPP_DROPIN),$(DI_DIR)/obj/$(call flat,$(s)).o)
DI_CU_OBJS := $(foreach s,$(CU_DROPIN),$(DI_DIR)/obj/$(call flat,$(s)).cu.o) $(DI_DIR)/obj/tensor__random.cu.o
DI_SHIM_CU_OBJS := $(DI_DIR)/obj/tt_runner_shim.cu.o $(DI_DIR)/obj/tt_conv_shim.cu.o $(DI_DIR)/obj/tt_reduce_all_shim.cu.o
DI_SHIM_OBJS := $(DI_SHIM_CU_OBJS) $(DI_DIR)/obj/tt_to_device_shim.o

# The reference's tests that pin the path and what sits either side of it.
TESTS_PLAIN := test_matmul test_multi_device_cuda test_to test_to_autograd test_clone test_rnn test_lstm test_gru
TESTS_TORCH := test_conv test_conv_autograd test_matmul_autograd
TEST_BINS := $(foreach t,$(TESTS_PLAIN) $(TESTS_TORCH),$(DI_DIR)/bin/$(t))

all: cpu dropin
cpu: $(CPU_DIR)/libtinytensor.a $(OUT)/libttref_full.so
dropin: $(DI_LIB) $(TEST_BINS)

$(GEN)/tt/export.h:
	mkdir -p $(GEN)/tt
	printf '#ifndef TINYTENSOR_EXPORT_H\n#define TINYTENSOR_EXPORT_H\n#define TINYTENSOR_EXPORT\n#define TINYTENSOR_NO_EXPORT\n#endif\n' > $@

# ---- CPU-only reference ------------------------------------------------------------------
define CPU_RULE
$(CPU_DIR)/obj/$(call flat,$(1)).o: $(REF)/tinytensor/$(1) $(GEN)/tt/export.h
	@mkdir -p $(CPU_DIR)/obj
	$(CXX) $(CXXFLAGS) -c $$< -o $$@
endef
$(foreach s,$(CPP_CPU),$(eval $(call CPU_RULE,$(s))))

$(CPU_DIR)/libtinytensor.a: $(CPU_OBJS)
	rm -f $@ && ar rcs $@ $^

# -Bsymbolic / --exclude-libs: where the toolchain links libstdc++ statically, the library must
# bind its own copy of the C++ runtime (exception handling above all) instead of whichever
# libstdc++ the loading process already holds.
$(OUT)/libttref_full.so: $(HERE)ref_full_driver.cpp $(CPU_DIR)/libtinytensor.a
	$(CXX) $(CXXFLAGS) -shared -Wl,-Bsymbolic -Wl,--exclude-libs,ALL -o $@ $< $(CPU_DIR)/libtinytensor.a

# ---- reference + CUDA backend with the matmul path swapped --------------------------------
DI_EXTRA_autograd__unary_ops := -DTensorToDevice=TensorToDeviceHostBounce
define DI_CPP_RULE
$(DI_DIR)/obj/$(call flat,$(1)).o: $(REF)/tinytensor/$(1) $(GEN)/tt/export.h $(HERE)dropin.mk
	@mkdir -p $(DI_DIR)/obj
	$(CXX) $(CXXFLAGS_BASE) -DTT_CUDA -I$(CUDA_HOME)/include $$(DI_EXTRA_$(call flat,$(1))) -c $$< -o $$@
endef
$(foreach s,$(CPP_DROPIN),$(eval $(call DI_CPP_RULE,$(s))))

DI_CUEXTRA_tensor__backend__cuda__conv := -Dbatched_conv2d_forward_runner=reference_conv2d_forward_runner \
	-Dbatched_conv2d_backward_runner=reference_conv2d_backward_runner
DI_CUEXTRA_tensor__backend__cuda__data_types := -include $(CSRC)/tt_alloc_shim.h
DI_CUEXTRA_tensor__backend__cuda__reduce := -Dreduce_all_runner=reference_reduce_all_runner
define DI_CU_RULE
$(DI_DIR)/obj/$(call flat,$(1)).cu.o: $(REF)/tinytensor/$(1) $(GEN)/tt/export.h $(CSRC)/tt_alloc_shim.h $(HERE)dropin.mk
	@mkdir -p $(DI_DIR)/obj
	$(NVCC) $(NVFLAGS) $$(DI_CUEXTRA_$(call flat,$(1))) -c $$< -o $$@
endef
$(foreach s,$(CU_DROPIN),$(eval $(call DI_CU_RULE,$(s))))

$(DI_DIR)/obj/tensor__random.cu.o: $(REF)/tinytensor/tensor/random.cpp $(GEN)/tt/export.h
	@mkdir -p $(DI_DIR)/obj
	$(NVCC) $(NVFLAGS) -x cu -c $< -o $@

$(DI_DIR)/obj/tt_%_shim.cu.o: $(CSRC)/tt_%_shim.cu $(ROOT)/include/ttb.h $(GEN)/tt/export.h
	@mkdir -p $(DI_DIR)/obj
	$(NVCC) $(NVFLAGS) -c $< -o $@

$(DI_DIR)/obj/tt_to_device_shim.o: $(CSRC)/tt_to_device_shim.cpp $(ROOT)/include/ttb.h $(GEN)/tt/export.h
	@mkdir -p $(DI_DIR)/obj
	$(CXX) $(CXXFLAGS_BASE) -DTT_CUDA -I$(CUDA_HOME)/include -c $< -o $@

# CUDA_RESOLVE_DEVICE_SYMBOLS ON (CMakeLists.txt:56-60): one device link of all relocatable objects.
$(DI_DIR)/obj/dlink.o: $(DI_CU_OBJS) $(DI_SHIM_CU_OBJS)
	$(NVCC) -gencode arch=compute_100a,code=sm_100a -dlink -Xcompiler -fPIC $^ -o $@

# $$ORIGIN-relative run path: oracle/_ref/tt_dropin -> the library is three levels up.
$(DI_LIB): $(DI_CPP_OBJS) $(DI_CU_OBJS) $(DI_SHIM_OBJS) $(DI_DIR)/obj/dlink.o $(LIBTTB)
	$(CXX) -shared -o $@ $(DI_CPP_OBJS) $(DI_CU_OBJS) $(DI_SHIM_OBJS) $(DI_DIR)/obj/dlink.o $(LIBTTB) \
	  -L$(CUDA_HOME)/lib64 -lcudart_static -ldl -lrt -lpthread -Wl,-rpath,'$$ORIGIN/../../../tinytensor_b200'

# ---- the reference's own tests against it -------------------------------------------------
TEST_CXXFLAGS := -std=c++20 -O2 -march=x86-64-v3 -DTT_CUDA -DTINYTENSOR_STATIC_DEFINE -w \
	-I$(REF)/include -I$(GEN) -I$(REF)/external/doctest -I$(REF)/tests
TEST_LDFLAGS := $(DI_LIB) $(LIBTTB) -Wl,-rpath,'$$ORIGIN/..' -Wl,-rpath,'$$ORIGIN/../../../../tinytensor_b200'
TORCH_CXXFLAGS := -DTT_TORCH -I$(TORCH_DIR)/include -I$(TORCH_DIR)/include/torch/csrc/api/include
TORCH_LDFLAGS := -L$(TORCH_DIR)/lib -Wl,--no-as-needed -ltorch -ltorch_cpu -lc10 -Wl,--as-needed -Wl,-rpath,$(TORCH_DIR)/lib

define PLAIN_TEST_RULE
$(DI_DIR)/bin/$(1): $(REF)/tests/$(1).cpp $(DI_LIB)
	@mkdir -p $(DI_DIR)/bin
	$(CXX) $(TEST_CXXFLAGS) $$< -o $$@ $(TEST_LDFLAGS)
endef
$(foreach t,$(TESTS_PLAIN),$(eval $(call PLAIN_TEST_RULE,$(t))))

define TORCH_TEST_RULE
$(DI_DIR)/bin/$(1): $(REF)/tests/$(1).cpp $(DI_LIB)
	@mkdir -p $(DI_DIR)/bin
	$(CXX) $(TEST_CXXFLAGS) $(TORCH_CXXFLAGS) $$< -o $$@ $(TEST_LDFLAGS) $(TORCH_LDFLAGS)
endef
$(foreach t,$(TESTS_TORCH),$(eval $(call TORCH_TEST_RULE,$(t))))

clean:
	rm -rf $(CPU_DIR) $(DI_DIR) $(OUT)/libttref_full.so

.PHONY: all cpu dropin clean

# Builds libuccl.so (host runtime + sm_100a kernels), the pybind11 module and the sample
# network plugin, all in-tree.  `make -j` is what __graft_entry__.build() runs.
CUDA_HOME ?= /usr/local/cuda
NVCC      ?= $(CUDA_HOME)/bin/nvcc
# Prefer the distribution compiler: it links libstdc++ dynamically, so the library shares the C++
# runtime of the process that loads it (a toolchain with only a static libstdc++ also works, the
# library code avoids iostreams for that case).
CXX       := $(firstword $(wildcard /usr/bin/g++) g++)
PYTHON    ?= python3

PYINC     := $(shell $(PYTHON) -c "import sysconfig; print(sysconfig.get_paths()['include'])")
PYBINDINC := $(shell $(PYTHON) -c "import pybind11; print(pybind11.get_include())")
EXTSUFFIX := $(shell $(PYTHON) -c "import sysconfig; print(sysconfig.get_config_var('EXT_SUFFIX'))")

BUILD     := build
PKG       := unified_ccl_b200
INCLUDES  := -Iinclude -Icsrc -I$(CUDA_HOME)/include
CXXFLAGS  := -O2 -g -std=c++17 -fPIC -Wall -Wno-unused-function -pthread $(INCLUDES)
NVFLAGS   := --extended-lambda -O3 -std=c++17 -lineinfo -gencode arch=compute_100a,code=sm_100a \
             -Xcompiler -fPIC,-Wall,-Wno-unused-function --expt-relaxed-constexpr $(INCLUDES)
LDFLAGS   := -shared -L$(CUDA_HOME)/lib64 -lcudart_static -ldl -lpthread -lrt

CC_SRCS := $(wildcard csrc/core/*.cc csrc/mem/*.cc csrc/transport/*.cc csrc/protocols/*.cc \
             csrc/rma/*.cc csrc/host/*.cc)
CU_SRCS := $(wildcard csrc/kernels/*.cu)
CC_OBJS := $(patsubst %.cc,$(BUILD)/%.o,$(CC_SRCS))
CU_OBJS := $(patsubst %.cu,$(BUILD)/%.cu.o,$(CU_SRCS))

LIB     := $(PKG)/libuccl.so
PYMOD   := $(PKG)/_uccl_bindings$(EXTSUFFIX)
PLUGIN  := plugins/sample/libuccl-net-sample.so

all: $(LIB) $(PYMOD) $(PLUGIN)

$(BUILD)/%.o: %.cc $(wildcard include/*.h csrc/*/*.h)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -c $< -o $@

$(BUILD)/%.cu.o: %.cu $(wildcard include/*.h csrc/*/*.h csrc/kernels/*.cuh)
	@mkdir -p $(dir $@)
	$(NVCC) $(NVFLAGS) -c $< -o $@

$(LIB): $(CC_OBJS) $(CU_OBJS)
	$(CXX) -o $@ $^ $(LDFLAGS)

$(PYMOD): csrc/python/bindings.cc $(LIB) $(wildcard include/*.h)
	$(CXX) $(CXXFLAGS) -fvisibility=hidden -I$(PYINC) -I$(PYBINDINC) -shared $< -o $@ \
	    -L$(PKG) -luccl -Wl,-rpath,'$$ORIGIN'

$(PLUGIN): plugins/sample/plugin.cc include/uccl_net.h include/uccl.h
	$(CXX) $(CXXFLAGS) -shared $< -o $@

# Host runtime under sanitizers: the native self tests (bootstrap, FIFO / proxy state machine,
# plugin loader, ring schedules, tuner, groups, CPU collectives) as a plain executable.
SAN_FLAGS_asan := -fsanitize=address,undefined -fno-omit-frame-pointer
SAN_FLAGS_tsan := -fsanitize=thread

define SAN_RULES
$(BUILD)/$(1)/%.o: %.cc $$(wildcard include/*.h csrc/*/*.h)
	@mkdir -p $$(dir $$@)
	$$(CXX) $$(filter-out -O2,$$(CXXFLAGS)) -O1 $$(SAN_FLAGS_$(1)) -c $$< -o $$@

$(BUILD)/$(1)/selftest: $$(patsubst %.cc,$(BUILD)/$(1)/%.o,$$(CC_SRCS)) $(BUILD)/$(1)/tests/native/selftest_main.o $$(CU_OBJS)
	$$(CXX) $$(SAN_FLAGS_$(1)) -o $$@ $$^ -L$$(CUDA_HOME)/lib64 -lcudart_static -ldl -lpthread -lrt

$(1): $(BUILD)/$(1)/selftest
	$(BUILD)/$(1)/selftest
endef
$(eval $(call SAN_RULES,asan))
$(eval $(call SAN_RULES,tsan))

clean:
	rm -rf $(BUILD) $(LIB) $(PYMOD) $(PLUGIN)

.PHONY: all clean asan tsan

# Builds libuccl.so (host runtime + sm_100a kernels), the pybind11 module, the sample network
# plugin and the test-only helper libraries, all in-tree.  `make -j` is what
# __graft_entry__.build() runs.
#
# Options (the reference's CMake switches, CMakeLists.txt:20-22, under the same names):
#   UCCL_BUILD_PYTHON=0      leave the pybind11 module out
#   UCCL_BUILD_TESTS=0       leave the test-only libraries (tests/native/) out
#   UCCL_BUILD_UCX_PLUGIN=1  build plugins/ucx/libuccl-net-ucx.so (needs UCX: UCX_HOME=<prefix>)
#   UCCL_BUILD_PLUGIN=0      leave the sample plugin out
# Install (the reference installs libuccl.so and its public headers, src/CMakeLists.txt:79-90):
#   make install PREFIX=/opt/uccl [DESTDIR=...]   ->  $(PREFIX)/lib/libuccl.so, $(PREFIX)/include/*.h
CUDA_HOME ?= /usr/local/cuda
NVCC      ?= $(CUDA_HOME)/bin/nvcc
# Prefer the distribution compiler: it links libstdc++ dynamically, so the library shares the C++
# runtime of the process that loads it (a toolchain with only a static libstdc++ also works, the
# library code avoids iostreams for that case).
CXX       := $(firstword $(wildcard /usr/bin/g++) g++)
PYTHON    ?= python3
PREFIX    ?= /usr/local
DESTDIR   ?=

UCCL_BUILD_PYTHON     ?= 1
UCCL_BUILD_TESTS      ?= 1
UCCL_BUILD_PLUGIN     ?= 1
UCCL_BUILD_UCX_PLUGIN ?= 0
UCX_HOME              ?= /usr

BUILD     := build
PKG       := unified_ccl_b200
INCLUDES  := -Iinclude -Icsrc -I$(CUDA_HOME)/include
CXXFLAGS  := -O2 -g -std=c++17 -fPIC -Wall -Wno-unused-function -pthread $(INCLUDES)
NVFLAGS   := --extended-lambda -O3 -std=c++17 -lineinfo -gencode arch=compute_100a,code=sm_100a \
             -Xcompiler -fPIC,-Wall,-Wno-unused-function --expt-relaxed-constexpr $(INCLUDES)
# UCCL_EXPERIMENTS=1 compiles the phase-skipping switches of the fused kernels in (see
# benchmarks/tp_breakdown.py); product builds leave them out.
ifeq ($(UCCL_EXPERIMENTS),1)
NVFLAGS   += -DUCCL_EXPERIMENTS=1
CXXFLAGS  += -DUCCL_EXPERIMENTS=1
endif
LDFLAGS   := -shared -L$(CUDA_HOME)/lib64 -lcudart_static -ldl -lpthread -lrt

CC_SRCS := $(wildcard csrc/core/*.cc csrc/mem/*.cc csrc/transport/*.cc csrc/protocols/*.cc \
             csrc/rma/*.cc csrc/host/*.cc)
CU_SRCS := $(wildcard csrc/kernels/*.cu)
CC_OBJS := $(patsubst %.cc,$(BUILD)/%.o,$(CC_SRCS))
CU_OBJS := $(patsubst %.cu,$(BUILD)/%.cu.o,$(CU_SRCS))

ifeq ($(UCCL_BUILD_PYTHON),1)
PYINC     := $(shell $(PYTHON) -c "import sysconfig; print(sysconfig.get_paths()['include'])")
PYBINDINC := $(shell $(PYTHON) -c "import pybind11; print(pybind11.get_include())")
EXTSUFFIX := $(shell $(PYTHON) -c "import sysconfig; print(sysconfig.get_config_var('EXT_SUFFIX'))")
endif
LIB       := $(PKG)/libuccl.so
PYMOD     := $(PKG)/_uccl_bindings$(EXTSUFFIX)
PLUGIN    := plugins/sample/libuccl-net-sample.so
UCXPLUGIN := plugins/ucx/libuccl-net-ucx.so
# test-only code: native self tests of the host runtime, kernels that call the device-side RMA
# API, and a C++ client of the C ABI
SELFTEST  := tests/native/libuccl_selftest.so
DEVTEST   := tests/native/libuccl_devtest.so
CLIENT    := tests/native/c_api_client
# one-pass SwiGLU of the NCCL + cuBLAS comparator (bench.py); not part of the library
BASELINE  := baseline/libbaseline_swiglu.so
PUBLIC_HEADERS := include/uccl.h include/uccl_net.h include/uccl_device.cuh include/uccl_noalloc.h

TARGETS := $(LIB) $(BASELINE)
ifeq ($(UCCL_BUILD_PYTHON),1)
TARGETS += $(PYMOD)
endif
ifeq ($(UCCL_BUILD_PLUGIN),1)
TARGETS += $(PLUGIN)
endif
ifeq ($(UCCL_BUILD_UCX_PLUGIN),1)
TARGETS += $(UCXPLUGIN)
endif
ifeq ($(UCCL_BUILD_TESTS),1)
TARGETS += $(SELFTEST) $(DEVTEST) $(CLIENT) plugins/ucx/libuccl-net-ucx-fake.so
endif

all: $(TARGETS)

$(BUILD)/%.o: %.cc $(wildcard include/*.h csrc/*/*.h)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -c $< -o $@

$(BUILD)/%.cu.o: %.cu $(wildcard include/*.h include/*.cuh csrc/*/*.h csrc/kernels/*.cuh)
	@mkdir -p $(dir $@)
	$(NVCC) $(NVFLAGS) -c $< -o $@

$(LIB): $(CC_OBJS) $(CU_OBJS)
	$(CXX) -o $@ $^ $(LDFLAGS)

$(PYMOD): csrc/python/bindings.cc $(LIB) $(wildcard include/*.h)
	$(CXX) $(CXXFLAGS) -fvisibility=hidden -I$(PYINC) -I$(PYBINDINC) -shared $< -o $@ \
	    -L$(PKG) -luccl -Wl,-rpath,'$$ORIGIN'

$(PLUGIN): plugins/sample/plugin.cc include/uccl_net.h include/uccl.h
	$(CXX) $(CXXFLAGS) -shared $< -o $@

# UCX transport plugin: real UCX when UCCL_BUILD_UCX_PLUGIN=1 (headers and libucp under UCX_HOME);
# `make ucx-fake` builds the same source against the in-tree stand-in of the few UCP calls it
# uses, which is what the CPU tests load.
$(UCXPLUGIN): plugins/ucx/plugin.cc include/uccl_net.h include/uccl.h
	$(CXX) $(CXXFLAGS) -DUCCL_HAS_UCX=1 -I$(UCX_HOME)/include -shared $< -o $@ -L$(UCX_HOME)/lib -lucp -lucs
plugins/ucx/libuccl-net-ucx-fake.so: plugins/ucx/plugin.cc plugins/ucx/fake_ucp.cc plugins/ucx/fake_ucp/ucp/api/ucp.h include/uccl_net.h include/uccl.h
	$(CXX) $(CXXFLAGS) -DUCCL_HAS_UCX=1 -Iplugins/ucx/fake_ucp -shared plugins/ucx/plugin.cc plugins/ucx/fake_ucp.cc -o $@
ucx-fake: plugins/ucx/libuccl-net-ucx-fake.so

$(SELFTEST): tests/native/selftest.cc tests/native/uccl_selftest.h $(LIB) $(wildcard include/*.h csrc/*/*.h)
	$(CXX) $(CXXFLAGS) -Itests/native -shared $< -o $@ -L$(PKG) -luccl -Wl,-rpath,'$$ORIGIN/../../$(PKG)'

$(DEVTEST): tests/native/rma_device_test.cu include/uccl_device.cuh include/uccl.h $(LIB)
	$(NVCC) $(NVFLAGS) -shared $< -o $@ -L$(PKG) -luccl -Xlinker -rpath,'$$ORIGIN/../../$(PKG)' -lcudart_static

$(BASELINE): baseline/swiglu_kernel.cu
	$(NVCC) $(NVFLAGS) -shared $< -o $@ -lcudart_static

$(CLIENT): tests/native/c_api_client.cc include/uccl.h $(LIB)
	$(CXX) $(CXXFLAGS) $< -o $@ -L$(PKG) -luccl -Wl,-rpath,'$$ORIGIN/../../$(PKG)' -L$(CUDA_HOME)/lib64 -lcudart_static -ldl -lpthread -lrt

install: $(LIB)
	install -d $(DESTDIR)$(PREFIX)/lib $(DESTDIR)$(PREFIX)/include
	install -m 755 $(LIB) $(DESTDIR)$(PREFIX)/lib/libuccl.so
	install -m 644 $(PUBLIC_HEADERS) $(DESTDIR)$(PREFIX)/include/
	install -d $(DESTDIR)$(PREFIX)/share/uccl/tuning
	install -m 644 $(PKG)/tuning/*.json $(DESTDIR)$(PREFIX)/share/uccl/tuning/
ifeq ($(UCCL_BUILD_PLUGIN),1)
	install -m 755 $(PLUGIN) $(DESTDIR)$(PREFIX)/lib/ 2>/dev/null || true
endif

# Host runtime under sanitizers: the native self tests (bootstrap, FIFO / proxy state machine,
# plugin loader, ring schedules, tuner, groups, CPU collectives) as a plain executable.
SAN_FLAGS_asan := -fsanitize=address,undefined -fno-omit-frame-pointer
SAN_FLAGS_tsan := -fsanitize=thread
SAN_SRCS := $(CC_SRCS) tests/native/selftest.cc tests/native/selftest_main.cc

define SAN_RULES
$(BUILD)/$(1)/%.o: %.cc $$(wildcard include/*.h csrc/*/*.h tests/native/*.h)
	@mkdir -p $$(dir $$@)
	$$(CXX) $$(filter-out -O2,$$(CXXFLAGS)) -Itests/native -O1 $$(SAN_FLAGS_$(1)) -c $$< -o $$@

$(BUILD)/$(1)/selftest: $$(patsubst %.cc,$(BUILD)/$(1)/%.o,$$(SAN_SRCS)) $$(CU_OBJS)
	$$(CXX) $$(SAN_FLAGS_$(1)) -o $$@ $$^ -L$$(CUDA_HOME)/lib64 -lcudart_static -ldl -lpthread -lrt

$(1): $(BUILD)/$(1)/selftest
	$(BUILD)/$(1)/selftest
endef
$(eval $(call SAN_RULES,asan))
$(eval $(call SAN_RULES,tsan))

clean:
	rm -rf $(BUILD) $(LIB) $(PYMOD) $(PLUGIN) $(SELFTEST) $(DEVTEST) $(CLIENT) $(BASELINE) plugins/ucx/*.so

.PHONY: all clean asan tsan install ucx-fake

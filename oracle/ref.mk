# Builds the UNMODIFIED reference (ggml core, ggml CPU backend, libllama and the
# reference's own test/bench tools) straight from its source files where they
# lie, into oracle/_ref/.  This is test infrastructure: the resulting CPU
# backend is the oracle the CUDA path is checked against and the timed CPU
# baseline.  No reference source is copied; the reference's own build system is
# not run.  Usage:   make -f oracle/ref.mk REF=/path/to/reference -j8   (REF defaults to a
# directory `reference` beside this repository)
#
# The ggml libraries are built in the reference's "dynamic backend" mode
# (GGML_BACKEND_DL): the CPU backend is produced as three loadable variants and
# the registry picks the best one the host CPU supports, so the same binaries
# run on the build container and on the GPU box's host.

REF   ?= $(abspath $(dir $(lastword $(MAKEFILE_LIST)))../../reference)
OUT  ?= oracle/_ref
OBJ  := $(OUT)/obj
CC   ?= gcc
CXX  ?= g++

GINC := -I$(REF)/ggml/include -I$(REF)/ggml/src
WARN := -w
COPT := -O3 -DNDEBUG -fPIC $(WARN) -D_GNU_SOURCE -D_XOPEN_SOURCE=600
CSTD := -std=gnu11
XSTD := -std=gnu++17

BASE_DEFS := -DGGML_BUILD -DGGML_SHARED -DGGML_SCHED_MAX_COPIES=4
BASE_C    := ggml.c ggml-alloc.c ggml-quants.c
BASE_CPP  := ggml-backend.cpp ggml-opt.cpp ggml-threading.cpp gguf.cpp
BASE_OBJS := $(addprefix $(OBJ)/base/,$(BASE_C:.c=.o) $(BASE_CPP:.cpp=.o))

REG_DEFS  := -DGGML_BUILD -DGGML_SHARED -DGGML_BACKEND_SHARED -DGGML_BACKEND_DL

CPU_DEFS  := -DGGML_BACKEND_BUILD -DGGML_BACKEND_SHARED -DGGML_BACKEND_DL -DGGML_SHARED \
             -DGGML_SCHED_MAX_COPIES=4 -DGGML_USE_CPU_AARCH64 -DGGML_USE_LLAMAFILE
CPU_INC   := $(GINC) -I$(REF)/ggml/src/ggml-cpu
CPU_C     := ggml-cpu.c ggml-cpu-quants.c
CPU_CPP   := ggml-cpu.cpp ggml-cpu-aarch64.cpp ggml-cpu-hbm.cpp ggml-cpu-traits.cpp \
             amx/amx.cpp amx/mmq.cpp llamafile/sgemm.cpp cpu-feats-x86.cpp

# variant -> arch flags / feature macros (the same sets the reference's
# GGML_CPU_ALL_VARIANTS list uses for these three names)
F_haswell := -msse4.2 -mf16c -mfma -mavx -mavx2
D_haswell := -DGGML_SSE42 -DGGML_F16C -DGGML_FMA -DGGML_AVX -DGGML_AVX2
F_icelake := $(F_haswell) -mavx512f -mavx512cd -mavx512vl -mavx512dq -mavx512bw -mavx512vbmi -mavx512vnni
D_icelake := $(D_haswell) -DGGML_AVX512 -DGGML_AVX512_VBMI -DGGML_AVX512_VNNI
F_sapphirerapids := $(F_icelake) -mavx512bf16 -mamx-tile -mamx-int8
D_sapphirerapids := $(D_icelake) -DGGML_AVX512_BF16 -DGGML_AMX_TILE -DGGML_AMX_INT8
VARIANTS := haswell icelake sapphirerapids

LLAMA_SRC := llama.cpp llama-adapter.cpp llama-arch.cpp llama-batch.cpp llama-chat.cpp \
             llama-context.cpp llama-grammar.cpp llama-hparams.cpp llama-impl.cpp \
             llama-kv-cache.cpp llama-mmap.cpp llama-model-loader.cpp llama-model.cpp \
             llama-quant.cpp llama-sampling.cpp llama-vocab.cpp unicode.cpp unicode-data.cpp
LLAMA_OBJS := $(addprefix $(OBJ)/llama/,$(LLAMA_SRC:.cpp=.o))
LLAMA_INC  := -I$(REF)/src -I$(REF)/include -I$(REF)/common -I$(REF)/ggml/include
LLAMA_DEFS := -DLLAMA_BUILD -DLLAMA_SHARED -DGGML_SHARED -DGGML_BACKEND_SHARED

COMMON_SRC := arg.cpp chat.cpp common.cpp console.cpp json-schema-to-grammar.cpp llguidance.cpp \
              log.cpp ngram-cache.cpp sampling.cpp speculative.cpp
COMMON_OBJS := $(addprefix $(OBJ)/common/,$(COMMON_SRC:.cpp=.o)) $(OBJ)/common/build-info.o
TOOL_INC   := -I$(REF)/common -I$(REF)/examples $(LLAMA_INC)
TOOL_DEFS  := -DLLAMA_SHARED -DGGML_SHARED -DGGML_BACKEND_SHARED
RPATH      := -Wl,-rpath,'$$ORIGIN'

CPU_LIBS := $(foreach v,$(VARIANTS),$(OUT)/libggml-cpu-$(v).so)

.PHONY: all core tools clean
all: core tools
core: $(OUT)/libggml-base.so $(OUT)/libggml.so $(CPU_LIBS) $(OUT)/test-backend-ops $(OUT)/test-quantize-fns
tools: $(OUT)/libllama.so $(OUT)/llama-bench $(OUT)/llama-quantize $(OUT)/llama-logits $(OUT)/graph-cases

# ---- ggml-base ----
$(OBJ)/base/%.o: $(REF)/ggml/src/%.c
	@mkdir -p $(dir $@)
	$(CC) $(COPT) $(CSTD) $(BASE_DEFS) $(GINC) -c $< -o $@
$(OBJ)/base/%.o: $(REF)/ggml/src/%.cpp
	@mkdir -p $(dir $@)
	$(CXX) $(COPT) $(XSTD) $(BASE_DEFS) $(GINC) -c $< -o $@
$(OUT)/libggml-base.so: $(BASE_OBJS)
	$(CXX) -shared -o $@ $^ -lm -lpthread

# ---- ggml (registry) ----
$(OBJ)/reg/ggml-backend-reg.o: $(REF)/ggml/src/ggml-backend-reg.cpp
	@mkdir -p $(dir $@)
	$(CXX) $(COPT) $(XSTD) $(REG_DEFS) $(GINC) -c $< -o $@
$(OUT)/libggml.so: $(OBJ)/reg/ggml-backend-reg.o $(OUT)/libggml-base.so
	$(CXX) -shared -o $@ $< -L$(OUT) -lggml-base -ldl $(RPATH)

# ---- CPU backend variants ----
define CPU_VARIANT
$(OBJ)/cpu-$(1)/%.c.o: $(REF)/ggml/src/ggml-cpu/%.c
	@mkdir -p $$(dir $$@)
	$(CC) $(COPT) $(CSTD) $(CPU_DEFS) $(D_$(1)) $(F_$(1)) $(CPU_INC) -c $$< -o $$@
$(OBJ)/cpu-$(1)/%.cpp.o: $(REF)/ggml/src/ggml-cpu/%.cpp
	@mkdir -p $$(dir $$@)
	$(CXX) $(COPT) $(XSTD) $(CPU_DEFS) $(D_$(1)) $(F_$(1)) $(CPU_INC) -c $$< -o $$@
$(OUT)/libggml-cpu-$(1).so: $(addprefix $(OBJ)/cpu-$(1)/,$(CPU_C:.c=.c.o) $(CPU_CPP:.cpp=.cpp.o)) $(OUT)/libggml-base.so
	$(CXX) -shared -o $$@ $$(filter %.o,$$^) -L$(OUT) -lggml-base -lm -lpthread -Wl,-rpath,'$$$$ORIGIN'
endef
$(foreach v,$(VARIANTS),$(eval $(call CPU_VARIANT,$(v))))

# ---- the reference's own tests against the backend ABI ----
$(OUT)/test-backend-ops: $(REF)/tests/test-backend-ops.cpp $(OUT)/libggml.so
	$(CXX) $(COPT) $(XSTD) $(TOOL_DEFS) -I$(REF)/ggml/include $< -o $@ -L$(OUT) -lggml -lggml-base -lpthread $(RPATH)
# (test-quantize-fns calls the CPU type traits directly, so it links the baseline CPU variant)
$(OUT)/test-quantize-fns: $(REF)/tests/test-quantize-fns.cpp $(OUT)/libggml.so $(OUT)/libggml-cpu-haswell.so
	$(CXX) $(COPT) $(XSTD) $(TOOL_DEFS) -I$(REF)/ggml/include -I$(REF)/ggml/src $< -o $@ -L$(OUT) -lggml -lggml-base -l:libggml-cpu-haswell.so -lpthread $(RPATH)

# ---- libllama + llama-bench (the unchanged callers of the backend ABI) ----
$(OBJ)/llama/%.o: $(REF)/src/%.cpp
	@mkdir -p $(dir $@)
	$(CXX) $(COPT) $(XSTD) $(LLAMA_DEFS) $(LLAMA_INC) -c $< -o $@
$(OUT)/libllama.so: $(LLAMA_OBJS) $(OUT)/libggml.so
	$(CXX) -shared -o $@ $(LLAMA_OBJS) -L$(OUT) -lggml -lggml-base -lpthread $(RPATH)

$(OBJ)/common/build-info.cpp:
	@mkdir -p $(dir $@)
	printf 'int LLAMA_BUILD_NUMBER = 0;\nchar const *LLAMA_COMMIT = "reference-snapshot";\nchar const *LLAMA_COMPILER = "gcc";\nchar const *LLAMA_BUILD_TARGET = "x86_64-linux";\n' > $@
$(OBJ)/common/build-info.o: $(OBJ)/common/build-info.cpp
	$(CXX) $(COPT) $(XSTD) -c $< -o $@
$(OBJ)/common/%.o: $(REF)/common/%.cpp
	@mkdir -p $(dir $@)
	$(CXX) $(COPT) $(XSTD) $(TOOL_DEFS) $(TOOL_INC) -c $< -o $@
$(OUT)/libcommon.a: $(COMMON_OBJS)
	ar rcs $@ $^

$(OUT)/llama-bench: $(REF)/examples/llama-bench/llama-bench.cpp $(OUT)/libcommon.a $(OUT)/libllama.so
	$(CXX) $(COPT) $(XSTD) $(TOOL_DEFS) $(TOOL_INC) $< -o $@ $(OUT)/libcommon.a -L$(OUT) -lllama -lggml -lggml-base -lpthread $(RPATH)
$(OUT)/llama-quantize: $(REF)/examples/quantize/quantize.cpp $(OUT)/libcommon.a $(OUT)/libllama.so
	$(CXX) $(COPT) $(XSTD) $(TOOL_DEFS) $(TOOL_INC) $< -o $@ $(OUT)/libcommon.a -L$(OUT) -lllama -lggml -lggml-base -lpthread $(RPATH)

# test tool of this repository (tests/native/llama_logits.cpp): libllama's public API only
$(OUT)/llama-logits: tests/native/llama_logits.cpp $(OUT)/libllama.so
	$(CXX) $(COPT) $(XSTD) $(TOOL_DEFS) $(TOOL_INC) $< -o $@ -L$(OUT) -lllama -lggml -lggml-base -lpthread $(RPATH)

# test tool of this repository (tests/native/graph_cases.cpp): hand-built graphs on the CPU backend and on a named device
$(OUT)/graph-cases: tests/native/graph_cases.cpp $(OUT)/libggml.so
	$(CXX) $(COPT) $(XSTD) $(TOOL_DEFS) -I$(REF)/ggml/include $< -o $@ -L$(OUT) -lggml -lggml-base -lpthread $(RPATH)

clean:
	rm -rf $(OUT)

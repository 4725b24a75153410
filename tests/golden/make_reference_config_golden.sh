#!/bin/sh
# Builds the reference's own host-side config parser (src/models/config.cpp with its JSON
# reader) with g++ and prints what it reads from the tiny test configurations, so that this
# repository's parser can be laid beside it.  Only the reference's host-only C++ compiles
# without ROCm; its model code (HIP) does not, which is why the numerics of the plain
# implementation rest on the reference's formulas rather than on its output.
#
#   sh tests/golden/make_reference_config_golden.sh /path/to/reference > tests/golden/reference_config.json
set -e
REF="${1:?path to the reference checkout}"
TMP="$(mktemp -d)"
python3 - "$TMP" <<'PY'
import json, os, sys
sys.path.insert(0, os.path.join(os.getcwd(), "tests"))
from tiny_configs import CONFIGS
for name, (cfg, _) in CONFIGS.items():
    json.dump(cfg, open(os.path.join(sys.argv[1], f"{name}.json"), "w"))
PY
cat > "$TMP/main.cpp" <<'CPP'
#include <cstdio>
#include "models/config.h"
int main(int argc, char** argv) {
  std::printf("{");
  for (int i = 1; i < argc; i += 2) {
    ninfer::ModelConfig c = ninfer::ModelConfig::from_file(argv[i + 1]);
    std::printf("%s\"%s\": {\"arch\": \"%s\", \"model_type\": \"%s\", \"vocab_size\": %d, \"hidden_size\": %d, "
                "\"num_hidden_layers\": %d, \"num_attention_heads\": %d, \"num_key_value_heads\": %d, "
                "\"intermediate_size\": %d, \"head_dim\": %d, \"rms_norm_eps\": %.9g, \"rope_theta\": %.9g, "
                "\"tie_word_embeddings\": %s, \"is_moe\": %s, \"num_experts\": %d, \"num_experts_per_tok\": %d, "
                "\"moe_intermediate_size\": %d, \"ffn_inner\": %d}",
                i > 1 ? ", " : "", argv[i], c.arch.c_str(), c.model_type.c_str(), c.vocab_size, c.hidden_size,
                c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.intermediate_size, c.head_dim,
                (double)c.rms_norm_eps, (double)c.rope_theta, c.tie_word_embeddings ? "true" : "false",
                c.is_moe ? "true" : "false", c.num_experts, c.num_experts_per_tok, c.moe_intermediate_size,
                c.ffn_inner());
  }
  std::printf("}\n");
  return 0;
}
CPP
g++ -std=c++17 -O1 -w -I"$REF/src" "$TMP/main.cpp" "$REF/src/models/config.cpp" "$REF/src/common/json.cpp" \
    "$REF/src/common/util.cpp" "$REF/src/common/log.cpp" -o "$TMP/refcfg"
"$TMP/refcfg" A "$TMP/A.json" B "$TMP/B.json" C "$TMP/C.json" 2>/dev/null
rm -r "$TMP"

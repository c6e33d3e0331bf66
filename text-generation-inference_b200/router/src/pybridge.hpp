// Embedded CPython bridge: tokenizer, chat templates and grammar compilation (router/pybridge.py).
// All calls are `json string -> json string`; the GIL is taken per call, so any thread may call.
#pragma once
#include <string>

#include "json.hpp"

namespace bridge {

// Starts the interpreter (once) and imports tgi_b200.router.pybridge; `repo_root` is put on sys.path.
void init(const std::string& repo_root);
void shutdown();
// Calls pybridge.<fn>(arg.dump()) and parses the reply; throws std::runtime_error on a Python error.
json::Value call(const char* fn, const json::Value& arg);

}  // namespace bridge

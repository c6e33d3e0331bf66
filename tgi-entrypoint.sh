#!/bin/bash
# Container entry point: refresh the linker cache (driver libraries are mounted at run time), then hand all
# arguments to the launcher.
ldconfig 2>/dev/null || true
exec tgi-b200-launcher "$@"

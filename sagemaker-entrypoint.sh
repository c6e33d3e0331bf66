#!/bin/bash
# SageMaker entry point.  The platform describes the deployment in environment variables, mounts an uploaded
# model under /opt/ml/model and expects the server on port 8080.  The launcher reads every flag from the
# environment as well (--num-shard <-> NUM_SHARD), so the platform's names only have to be translated.
set -u
declare -A translate=(
  [HF_MODEL_ID]=MODEL_ID
  [HF_MODEL_REVISION]=REVISION
  [HF_MODEL_QUANTIZE]=QUANTIZE
  [HF_MODEL_TRUST_REMOTE_CODE]=TRUST_REMOTE_CODE
  [SM_NUM_GPUS]=NUM_SHARD
)
for platform_name in "${!translate[@]}"; do
  value="${!platform_name:-}"
  [[ -n "$value" ]] && export "${translate[$platform_name]}=$value"
done
if [[ -z "${MODEL_ID:-}" ]]; then
  if [[ -d /opt/ml/model ]]; then
    export MODEL_ID=/opt/ml/model
  else
    echo "sagemaker-entrypoint: set HF_MODEL_ID or mount a model at /opt/ml/model" >&2
    exit 64
  fi
fi
ldconfig 2>/dev/null || true
exec tgi-b200-launcher --port 8080 "$@"

#!/bin/bash
# SageMaker entry point: the platform passes configuration in environment variables and expects the server on
# port 8080 with the model under /opt/ml/model (or a hub id in HF_MODEL_ID).
if [[ -z "${HF_MODEL_ID}" ]]; then
  if [[ -d /opt/ml/model ]]; then
    export HF_MODEL_ID=/opt/ml/model
  else
    echo "HF_MODEL_ID must be set" >&2
    exit 1
  fi
fi
export MODEL_ID="${HF_MODEL_ID}"
if [[ -n "${HF_MODEL_REVISION}" ]]; then export REVISION="${HF_MODEL_REVISION}"; fi
if [[ -n "${SM_NUM_GPUS}" ]]; then export NUM_SHARD="${SM_NUM_GPUS}"; fi
if [[ -n "${HF_MODEL_QUANTIZE}" ]]; then export QUANTIZE="${HF_MODEL_QUANTIZE}"; fi
if [[ -n "${HF_MODEL_TRUST_REMOTE_CODE}" ]]; then export TRUST_REMOTE_CODE="${HF_MODEL_TRUST_REMOTE_CODE}"; fi
ldconfig 2>/dev/null || true
exec tgi-b200-launcher --port 8080 "$@"

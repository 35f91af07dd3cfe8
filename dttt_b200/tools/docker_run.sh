#!/usr/bin/env bash
# Launch a command (default: the image's shell) inside the training container on a GPU node.
#
#   dttt_b200/tools/docker_run.sh python -m dttt_b200.train --config runs/trunk_8k.json
#
# The container runs as the calling user (files on the mounts stay the user's, and signals sent on the host reach
# the training process), shares the host's network and IPC namespaces (NCCL, CUDA IPC between the ranks of a node),
# sees every GPU, and gets the repository, checkpoints, logs and token streams as bind mounts.  Environment variables
# whose names start with NCCL_, DTTT_, TTT_, TORCH_, CUDA_ or WANDB_ are forwarded BY NAME, so secrets never show up on a
# command line.  Settings (all optional, from the environment):
#   IMAGE_NAME   image to run                      (dttt-b200:latest)
#   CODE_DIR     repository on the host            (the checkout this script lives in)
#   DATA_DIR     token streams                     ($CODE_DIR/data/tokens; mounted read-only when it exists)
#   CKPT_DIR     checkpoints                       ($CODE_DIR/ckpt)
#   LOG_DIR      logs and evaluation files         ($CODE_DIR/log)
# Role of the reference's tools/docker_run.sh.
set -euo pipefail

here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
repo="$(cd "${here}/../.." && pwd)"
command -v docker >/dev/null 2>&1 || { echo "docker_run: docker is not on PATH" >&2; exit 1; }

image="${IMAGE_NAME:-dttt-b200:latest}"
code="${CODE_DIR:-${repo}}"
data="${DATA_DIR:-${code}/data/tokens}"
ckpt="${CKPT_DIR:-${code}/ckpt}"
logs="${LOG_DIR:-${code}/log}"

# mount sources must exist (and belong to the user) before the runtime would create them as root
mkdir -p "${ckpt}" "${logs}" "${code}/ckpt" "${code}/log"

args=(--rm --init --ipc=host --net=host --gpus all --user "$(id -u):$(id -g)" -e HOME=/tmp -e USER
      --ulimit memlock=-1:-1 --ulimit stack=67108864 -w /workspace
      -v "${code}:/workspace" -v "${ckpt}:/workspace/ckpt" -v "${logs}:/workspace/log")
for gid in $(id -G); do args+=(--group-add "${gid}"); done
while IFS= read -r name; do args+=(-e "${name}"); done < <(compgen -e | grep -E '^(NCCL_|DTTT_|TTT_|TORCH_|WANDB_)|^CUDA_VISIBLE_DEVICES$' || true)

if [[ -d /dev/infiniband ]]; then
  args+=(--device /dev/infiniband)
  echo "[docker_run] network: /dev/infiniband passed through (multi-node NCCL over IB / RoCE)" >&2
else
  echo "[docker_run] network: no /dev/infiniband; NCCL uses NVLink inside the node and TCP between nodes" >&2
fi
if [[ -d "${data}" ]]; then
  mkdir -p "${code}/data/tokens"
  args+=(-v "${data}:/workspace/data/tokens:ro")
  echo "[docker_run] data:    ${data} -> /workspace/data/tokens (read-only)" >&2
else
  echo "[docker_run] data:    ${data} does not exist; not mounted" >&2
fi
[[ -t 0 && -t 1 ]] && args+=(-it)

echo "[docker_run] image ${image}; code ${code}; checkpoints ${ckpt}; logs ${logs}" >&2
exec docker run "${args[@]}" "${image}" "$@"

#!/bin/bash
#SBATCH --job-name={{ job_name }}
#SBATCH --nodes={{ nodes }}
#SBATCH --ntasks-per-node=1
#SBATCH --gres=gpu:{{ n_proc_per_node }}
#SBATCH --cpus-per-task=32
#SBATCH --time={{ time_limit }}
#SBATCH --output={{ root_path }}/log_%j.out
#SBATCH --error={{ root_path }}/log_%j.out
{% if qos %}#SBATCH --qos={{ qos }}{% endif %}

# One training run of picotron_b200. The status file next to the config follows
# init -> pending -> running -> {completed, fail, oom, timeout}.
set -u
STATUS_FILE={{ root_path }}/status.txt
echo running > "$STATUS_FILE"

export CUDA_DEVICE_MAX_CONNECTIONS=1
export OMP_NUM_THREADS=1
MASTER_NODE=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
MASTER_PORT=$((20000 + SLURM_JOB_ID % 20000))

srun torchrun --nnodes={{ nodes }} --nproc_per_node={{ n_proc_per_node }} --max_restarts 0 --tee 3 \
    --rdzv_backend c10d --rdzv_endpoint "$MASTER_NODE:$MASTER_PORT" \
    {{ repo_path }}/train.py --config {{ config }}
RC=$?

LOG={{ root_path }}/log_${SLURM_JOB_ID}.out
if [ $RC -eq 0 ]; then
    echo completed > "$STATUS_FILE"
elif grep -q "OutOfMemoryError" "$LOG"; then
    echo oom > "$STATUS_FILE"
elif grep -qi "timeout\|watchdog" "$LOG"; then
    echo timeout > "$STATUS_FILE"
else
    echo fail > "$STATUS_FILE"
fi
exit $RC

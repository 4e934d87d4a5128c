# Single-process training on a Windows workstation (CPU or one GPU).  Multi-GPU launches go through scripts/bash/distributed.sh.
param(
    [string]$Config = "configs/train_single.yaml",
    [string]$ModelConfig = "",
    [ValidateSet("auto", "cpu", "cuda")][string]$Device = "auto",
    [string]$Resume = "",
    [int]$SmokeSteps = 0,
    [string]$Python = $(if ($env:PYTHON) { $env:PYTHON } else { "python" })
)
$ErrorActionPreference = "Stop"
$Root = Split-Path -Parent (Split-Path -Parent $PSScriptRoot)
Set-Location $Root
$TrainArgs = @("scripts/train.py", "--config", $Config, "--device", $Device)
if ($ModelConfig) { $TrainArgs += @("--model-config", $ModelConfig) }
if ($Resume) { $TrainArgs += @("--resume", $Resume) }
if ($SmokeSteps -gt 0) { $TrainArgs += @("--smoke-steps", "$SmokeSteps") }
& $Python @TrainArgs
if ($LASTEXITCODE -ne 0) { exit $LASTEXITCODE }

# Remove Python byte-code caches and pytest / hypothesis state; the built extension and its build directory are kept.
$ErrorActionPreference = "Stop"
$Root = Split-Path -Parent (Split-Path -Parent $PSScriptRoot)
Get-ChildItem -LiteralPath $Root -Directory -Recurse -Force |
    Where-Object { $_.Name -in "__pycache__", ".pytest_cache", ".hypothesis" } |
    Remove-Item -Recurse -Force
Get-ChildItem -LiteralPath $Root -File -Recurse -Force |
    Where-Object { $_.Extension -in ".pyc", ".pyo" } |
    Remove-Item -Force
Write-Host "Python caches removed; mini_train_sys_b200/_build and the extension binary were kept."

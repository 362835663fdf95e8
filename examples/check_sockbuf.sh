#!/usr/bin/env bash
# Prints the kernel's socket-buffer limits next to what the host transport asks for
# (MCCL_SOCK_BUFSIZE, default 4 MiB): a limit below the request silently caps the TCP window of the
# CPU-tensor path and of the host-staged fallback.
set -euo pipefail
want=${MCCL_SOCK_BUFSIZE:-4194304}
for k in net.core.rmem_max net.core.wmem_max; do
  v=$(sysctl -n "$k" 2>/dev/null || echo unknown)
  if [ "$v" != unknown ] && [ "$v" -lt "$want" ]; then note="  < requested $want: raise with 'sysctl -w $k=$want'"; else note=""; fi
  echo "$k = $v$note"
done
sysctl -n net.ipv4.tcp_rmem net.ipv4.tcp_wmem 2>/dev/null | sed 's/^/tcp_{r,w}mem: /' || true

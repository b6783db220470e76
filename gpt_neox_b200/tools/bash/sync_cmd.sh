#!/usr/bin/env bash
# Run one command on every host of the hostfile.  usage: sync_cmd.sh '<command>' [hostfile]
CMD=$1; HOSTFILE=${2:-/job/hostfile}
pdsh -f 1024 -R ssh -w "$(awk '{print $1}' "$HOSTFILE" | paste -sd, -)" "$CMD"

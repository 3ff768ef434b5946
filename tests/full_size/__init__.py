/bin/bash: line 1: unalias: bq: not found

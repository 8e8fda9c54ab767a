"""``python -m cornserve.services.pb [dir]`` writes the ``.proto`` files generated from the schema table."""

import sys

from . import write_proto_files

for path in write_proto_files(sys.argv[1] if len(sys.argv) > 1 else "proto/v1"):
    print("wrote", path)

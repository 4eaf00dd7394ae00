import sys

from lily_b200.entrypoints.cli import main

sys.exit(main())

import sys

from atomserve_b200.engine.cli import main

sys.exit(main())

import sys

from aklr_b200.csrc.probes import main

sys.exit(main())

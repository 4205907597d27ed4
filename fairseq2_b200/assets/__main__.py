import sys

from fairseq2_b200.assets.cli import main

sys.exit(main())

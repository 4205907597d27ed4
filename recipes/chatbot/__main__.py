import sys

from .program import main

sys.exit(main())

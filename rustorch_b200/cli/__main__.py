import sys

from .repl import main

sys.exit(main())

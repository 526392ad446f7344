"""Name used by the reference for its serial validation script; the implementation is ``serial.py``."""

from serial import main

if __name__ == "__main__":
    main()

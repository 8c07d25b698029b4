"""CPU checker for the flash_dism hard path: test infrastructure, never a product path."""

"""TEST INFRASTRUCTURE.  CPU oracle of the chunk optimizer step; see ``elx_oracle.c``."""

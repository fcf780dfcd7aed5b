"""CPU oracle for the NVFP4 linear path: TEST INFRASTRUCTURE, never imported by the product."""

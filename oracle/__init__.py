"""CPU checkers for the sampler.  TEST INFRASTRUCTURE ONLY -- never imported by the product.

``oracle.c_oracle``   fp32, operation-order-faithful C restatement of the reference kernels
``oracle.cpu_ref``    float64 torch statement of the same sampling semantics (sort + cumsum)
``oracle.philox_py``  pure-Python Philox4x32-10 for known-answer tests
``oracle.build_ref``  recipe that compiles the reference's own CUDA extension into oracle/_ref/
"""

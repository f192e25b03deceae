"""CPU oracle (test infrastructure): numpy restatement `ztvm_oracle`, C twin `ztvm_oracle_c`."""

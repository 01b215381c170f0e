/* empty: the reference only uses cblas under #ifdef OPENBLAS */

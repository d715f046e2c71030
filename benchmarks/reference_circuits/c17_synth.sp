* c17, all inputs high: 6 gates, 24 transistors
VDD vdd 0 DC 1.8
VIN0 n1 0 DC 1.8
VIN1 n2 0 DC 1.8
VIN2 n3 0 DC 1.8
VIN3 n6 0 DC 1.8
VIN4 n7 0 DC 1.8
M1 n10 n1 vdd vdd pch w=2u l=180n
M2 n10 n3 vdd vdd pch w=2u l=180n
CT1 t1 0 0.1f
M3 n10 n1 t1 0 nch w=1u l=180n
M4 t1 n3 0 0 nch w=1u l=180n
Cn10 n10 0 2f
M5 n11 n3 vdd vdd pch w=2u l=180n
M6 n11 n6 vdd vdd pch w=2u l=180n
CT2 t2 0 0.1f
M7 n11 n3 t2 0 nch w=1u l=180n
M8 t2 n6 0 0 nch w=1u l=180n
Cn11 n11 0 2f
M9 n16 n2 vdd vdd pch w=2u l=180n
M10 n16 n11 vdd vdd pch w=2u l=180n
CT3 t3 0 0.1f
M11 n16 n2 t3 0 nch w=1u l=180n
M12 t3 n11 0 0 nch w=1u l=180n
Cn16 n16 0 2f
M13 n19 n11 vdd vdd pch w=2u l=180n
M14 n19 n7 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M15 n19 n11 t4 0 nch w=1u l=180n
M16 t4 n7 0 0 nch w=1u l=180n
Cn19 n19 0 2f
M17 n22 n10 vdd vdd pch w=2u l=180n
M18 n22 n16 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M19 n22 n10 t5 0 nch w=1u l=180n
M20 t5 n16 0 0 nch w=1u l=180n
Cn22 n22 0 2f
M21 n23 n16 vdd vdd pch w=2u l=180n
M22 n23 n19 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M23 n23 n16 t6 0 nch w=1u l=180n
M24 t6 n19 0 0 nch w=1u l=180n
Cn23 n23 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: n22 n23
.end
